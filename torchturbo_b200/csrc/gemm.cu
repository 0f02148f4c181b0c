// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared (128B swizzle)
// -> tcgen05.mma (cta_group::1, M=128) -> TMEM (double-buffered accumulator)
// -> tcgen05.ld epilogue.  One kernel body covers
//   * dense  C[M,N] = A . B          with A / B each K-major or MN-major in memory,
//   * grouped-M (MoE forward / dX): rows are grouped by expert in 128-row aligned
//     segments, `tile_group[m_tile]` names the expert whose B[g] the tile uses
//     (-1 skips the tile).  Offsets live on the device; the host never syncs.
//   * grouped-K (MoE dW): C[g] = A[rows_g]^T . B[rows_g] with row ranges from a
//     device array (64-aligned, pad rows are zero).
// Epilogues: plain store (bf16 or fp32, optional accumulate / residual add) and
// SwiGLU (gate and up column panels are loaded side by side into one 256-wide
// accumulator; out = silu(g) * u * row_scale, pre-activations optionally kept).
//
//
// Expert-parallel fusion (grouped-M only, both optional, see `EpFuse`):
//   * push prologue: two extra warps per CTA copy this rank's routed token rows (plus routing weight and a
//     return tag) straight into the owning ranks' expert-major receive buffers over NVLink while the tensor
//     cores work; rows travel in (local expert, owner) order and every (source, expert) pair raises a flag on
//     the owner when its last row has landed.  The TMA producer warp waits (bounded) for the flags of a
//     tile's expert the first time the CTA meets it, so the math of the first experts overlaps the transfer
//     of the later ones.  This is the token dispatch all-to-all of the reference
//     (models/modules/moe/token_dispatcher.py:149-201) inside the fc1 GEMM.
//   * scatter epilogue: every output row is stored straight into the source rank's [T*k, N] return buffer at
//     the position its tag names (peer stores from the epilogue warps); the last CTA raises a "rows
//     returned" flag on every peer.  This is the combine all-to-all (token_dispatcher.py:203-236) inside the
//     fc2 / input-gradient GEMM.
//
// Replaces cuBLAS `F.linear`, `grouped_gemm.ops.gmm` and the torch.compile'd
// SwiGLU of the reference (ops/providers/cuda/grouped_matmul.py:19-36,
// ops/providers/cuda/swiglu.py:26-36, models/modules/moe/experts.py:181-254).
#include "peer.cuh"
#include <cstring>

namespace ttb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr unsigned KID_GEMM = 1;

enum Epi : int { EPI_STORE = 0, EPI_SWIGLU = 1 };

// Expert-parallel fusion parameters (device side).
struct EpFuse {
  PeerTable peers;
  // push prologue
  int push_on;
  long long off_rows, off_vals, off_tags, off_flags;  // byte offsets inside every rank's symmetric buffer
  const __nv_bfloat16* src;   // [T, lds] local token rows
  long long lds;
  const int* order;           // [n_entries] entry ids (token * k + slot) in send order
  const int* expert;          // [n_entries] global expert of every entry
  const int* dest_row;        // [n_entries] row on the owner
  const float* val;           // [n_entries] scalar that travels with the row, or null
  const int* counts;          // [E] rows this rank sends per global expert
  int* sent;                  // [E + 1] rows sent per expert, then the next chunk to claim; all zero at launch
  int n_entries, k, H, El, W, rank, epoch;
  long long cap_rows;
  unsigned long long budget_ns;
  int* status;
  // scatter epilogue
  int scat_on;
  long long off_ret, off_ret_vals, off_ret_flags;
  const int* row_tag;         // [M] tags of this rank's received rows
  const float* row_val;       // [M] scalar returned with the row, or null
  int ret_epoch;
  unsigned int* done_counter;
  int ret_rows;               // rows of every rank's return buffer (tags at or past it are refused)
};

struct GemmParams {
  EpFuse ep;
  int M, N, K;   // per-problem extents (N = output columns; for SwiGLU N = F)
  int m_tiles, n_tiles, groups_k;  // groups_k > 0 => grouped-K problem count
  void* C;
  long long ldc;         // elements
  long long c_group_stride;  // elements between C[g] (grouped-K)
  int c_fp32;            // 1: fp32 output, 0: bf16
  int accumulate;        // C += result (read-modify-write)
  const __nv_bfloat16* residual;  // optional [M, ldr] added before store (bf16 out)
  long long ldr;
  const int* tile_group;  // grouped-M: [m_tiles]
  const int* group_rows;  // grouped-K: [groups_k + 1], multiples of BK
  // SwiGLU
  int F;                  // gate columns [0,F), up columns [F,2F)
  const float* row_scale; // optional [M]
  __nv_bfloat16* preact;  // optional [M, ld_preact] receives gate|up
  long long ld_preact;
};

template <int BN, bool A_MN, bool B_MN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int EPI_STAGE_BYTES = 32 * 32 * 4;   // one 32-row x 32-column fp32 chunk per epilogue warp
  static constexpr int EPI_BYTES = 8 * EPI_STAGE_BYTES;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

constexpr int EPI_WARPS = 8;                       // two warps per TMEM lane quarter, each takes half of the columns
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int PUSH_WARPS = 2;                      // extra warps of a launch with the push prologue
constexpr int GEMM_THREADS_PUSH = GEMM_THREADS + 32 * PUSH_WARPS;
constexpr int PUSH_CHUNK = 8;                      // rows a push warp copies between two system-scope fences
static_assert(EPI_WARPS == 8, "the staging area is sized for eight epilogue warps");

// Epilogue staging.  tcgen05.ld hands every lane 32 consecutive columns of ITS row, so direct stores touch 32 rows per
// instruction with 16 bytes each.  The chunk is instead parked in shared memory (fp32, 128 bytes per row, 16-byte
// pieces XOR-swizzled by the row so that neither side has more than the unavoidable 4-way bank split) and written
// out row-major: one instruction stores whole 64-byte (bf16) or 128-byte (fp32) row segments of 8 or 4 rows.
__device__ __forceinline__ uint32_t epi_piece_addr(uint32_t base, int row, int piece) {
  return base + row * 128 + ((piece ^ (row & 7)) << 4);
}
// same for packed bf16 chunks: 64 bytes per row, four 16-byte pieces
__device__ __forceinline__ uint32_t epi_piece_addr64(uint32_t base, int row, int piece) {
  return base + row * 64 + ((piece ^ ((row >> 1) & 3)) << 4);
}

template <int BN, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS_PUSH, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  using L = SmemLayout<BN, A_MN, B_MN>;
  constexpr int STAGES = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + STAGES * L::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * L::STAGE_BYTES + L::EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  __shared__ uint32_t s_landed[32];   // push prologue: experts (up to 1024) whose rows are known to have landed
  __shared__ int s_last_cta;
  __shared__ int s_dead;              // the exchange this launch belongs to has already failed: no tile is computed

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // With the push prologue the producer may spend up to the exchange budget waiting for a peer's rows; the warps
  // downstream of it (MMA issuer, epilogue) must outwait it, or they give up on tiles whose rows arrive later.
  const uint64_t consumer_budget = p.ep.push_on ? p.ep.budget_ns + kWaitBudgetNs : kWaitBudgetNs;

  if (threadIdx.x < 32) s_landed[threadIdx.x] = 0u;
  if (threadIdx.x == 0) {
    // rows of a failed exchange never arrive: without this every CTA would sit out the full wait budget per launch
    s_dead = (p.ep.status != nullptr && *reinterpret_cast<volatile int*>(p.ep.status) != 0) ? 1 : 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], EPI_WARPS);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int groups = p.groups_k > 0 ? p.groups_k : 1;
  const long long tiles_per_group = static_cast<long long>(p.m_tiles) * p.n_tiles;
  const long long total_tiles = s_dead ? 0 : tiles_per_group * groups;

  // Decode tile -> (g, m_tile, n_tile).  Tiles are walked in bands of RASTER_M m-tiles: inside a band m runs
  // fastest, then n, so the ~148 tiles in flight cover a near-square RASTER_M x (148 / RASTER_M) block of C.  Per wave
  // that needs RASTER_M A panels and ~9 B panels instead of every A panel, and a band's A panels stay in L2 while
  // its n-tiles are walked (an m-fastest walk over all m-tiles re-read A from DRAM once per n-tile column).
  constexpr int RASTER_M = 16;
  auto decode = [&](long long t, int& g, int& mt, int& nt) {
    g = static_cast<int>(t / tiles_per_group);
    const long long r = t - static_cast<long long>(g) * tiles_per_group;
    const long long per_band = static_cast<long long>(RASTER_M) * p.n_tiles;
    const int band = static_cast<int>(r / per_band);
    const int m_base = band * RASTER_M;
    const int band_rows = (p.m_tiles - m_base) < RASTER_M ? (p.m_tiles - m_base) : RASTER_M;
    const long long w = r - static_cast<long long>(band) * per_band;
    nt = static_cast<int>(w / band_rows);
    mt = m_base + static_cast<int>(w - static_cast<long long>(nt) * band_rows);
  };
  // k-range of a tile: dense -> [0, K); grouped-K -> rows of group g.
  auto krange = [&](int g, int& k0, int& nkb) {
    if (p.groups_k > 0) {
      int r0 = p.group_rows[g], r1 = p.group_rows[g + 1];
      k0 = r0;
      nkb = (r1 - r0) / BK;
    } else {
      k0 = 0;
      nkb = (p.K + BK - 1) / BK;
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    // all k-blocks of one tile; run by one thread
    auto load_tile = [&](int g, int mt, int nt, int bgroup) -> bool {
      int k0, nkb;
      krange(g, k0, nkb);
      const int m0 = mt * BM;
      const int n0 = nt * (EPI == EPI_SWIGLU ? BN / 2 : BN);
      for (int kb = 0; kb < nkb; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, KID_GEMM, 1)) return false;
        uint8_t* sa = smem + stage * L::STAGE_BYTES;
        uint8_t* sb = sa + L::A_BYTES;
        mbar_expect_tx(&full[stage], L::STAGE_BYTES);
        const int kc = k0 + kb * BK;
        if (!A_MN) {
          tma_load_2d(sa, &tmA, &full[stage], kc, m0);
        } else {
          tma_load_2d(sa, &tmA, &full[stage], m0, kc);
          tma_load_2d(sa + 8192, &tmA, &full[stage], m0 + 64, kc);
        }
        if (!B_MN) {
          if (EPI == EPI_SWIGLU) {
            tma_load_3d(sb, &tmB, &full[stage], kc, n0, bgroup);
            tma_load_3d(sb + (BN / 2) * 128, &tmB, &full[stage], kc, p.F + n0, bgroup);
          } else {
            tma_load_3d(sb, &tmB, &full[stage], kc, n0, bgroup);
          }
        } else {
          constexpr int PANELS = BN / 64;
#pragma unroll
          for (int q = 0; q < PANELS; ++q) {
            int nc;
            if (EPI == EPI_SWIGLU) {
              nc = (q < PANELS / 2) ? (n0 + q * 64) : (p.F + n0 + (q - PANELS / 2) * 64);
            } else {
              nc = n0 + q * 64;
            }
            tma_load_3d(sb + q * 8192, &tmB, &full[stage], nc, kc, bgroup);
          }
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      return true;
    };
    if (!p.ep.push_on) {
      if (elect_one()) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
          int g, mt, nt;
          decode(t, g, mt, nt);
          int bgroup = 0;
          if (p.tile_group) {
            bgroup = p.tile_group[mt];
            if (bgroup < 0) continue;
          }
          if (!load_tile(g, mt, nt, bgroup)) break;
        }
      }
    } else {
      // Push prologue active: the rows of A arrive from the peers while this kernel runs.  The whole warp walks the
      // tile list; the first time the CTA meets an expert, lane s waits (bounded) for "source s has delivered its
      // rows of this expert", then lane 0 issues the tile's loads.
      if (lane == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
      }
      const int* my_flags = reinterpret_cast<const int*>(p.ep.peers.base[p.ep.rank] + p.ep.off_flags);
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int g, mt, nt;
        decode(t, g, mt, nt);
        const int bgroup = p.tile_group[mt];
        if (bgroup < 0) continue;
        if (!((s_landed[bgroup >> 5] >> (bgroup & 31)) & 1u)) {
          bool mine = true;
          if (lane < p.ep.W)
            mine = wait_flag(my_flags + bgroup * p.ep.W + lane, p.ep.epoch, p.ep.budget_ns, 9, lane, p.ep.status);
          ok = __all_sync(0xffffffffu, mine);
          if (!ok) break;
          if (lane == 0) s_landed[bgroup >> 5] |= 1u << (bgroup & 31);
          __syncwarp();
        }
        if (lane == 0) {
          fence_proxy_async_all();
          ok = load_tile(g, mt, nt, bgroup);
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int g, mt, nt, k0, nkb;
        decode(t, g, mt, nt);
        if (p.tile_group && p.tile_group[mt] < 0) continue;
        krange(g, k0, nkb);
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, KID_GEMM, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full[stage], phase, KID_GEMM, 3, consumer_budget)) {
            if (p.ep.status) atomicCAS(p.ep.status, 0, 0x10000 | (11 << 8));
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc(sa + kk * 2048, 8192, 1024)
                                     : make_smem_desc(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + kk * 2048, 8192, 1024)
                                     : make_smem_desc(sb + kk * 32, 16, 1024);
            umma_ss(d_tmem, da, db, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    const int lane_group = warp & 3;  // TMEM lanes [32*lane_group, +32) are the ones this warp may touch
    const int col_half = (warp - 2) >> 2;  // which half of the tile's column chunks this warp stores
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int g, mt, nt, k0, nkb;
      decode(t, g, mt, nt);
      if (p.tile_group && p.tile_group[mt] < 0) continue;
      krange(g, k0, nkb);
      if (!mbar_wait(&tfull[acc], acc_phase, KID_GEMM, 4, consumer_budget)) { ok = false; break; }
      tc_fence_after();
      const int row = mt * BM + lane_group * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(lane_group * 32) << 16);

      if (EPI == EPI_STORE) {
        const int n0 = nt * BN;
        uint8_t* cbase = reinterpret_cast<uint8_t*>(p.C);
        const long long coff = static_cast<long long>(g) * p.c_group_stride + static_cast<long long>(row) * p.ldc;
        // bf16 output: first element of the four rows this lane stores in the row-major pass (null = skip the row).
        // With the scatter epilogue a row goes to the rank it came from, at the entry its tag names.
        __nv_bfloat16* rowptr[4] = {nullptr, nullptr, nullptr, nullptr};
        if (!p.c_fp32) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int rr = mt * BM + lane_group * 32 + (lane >> 2) + 8 * j;
            if (rr >= p.M) continue;
            if (p.ep.scat_on) {
              const int tag = __ldcg(p.ep.row_tag + rr);
              if (tag >= 0) {
                // a tag that names no rank or no entry (rows that never landed) must not become an address
                if ((tag >> EP_TAG_SHIFT) < p.ep.W && (tag & EP_TAG_MASK) < p.ep.ret_rows)
                  rowptr[j] = reinterpret_cast<__nv_bfloat16*>(p.ep.peers.base[tag >> EP_TAG_SHIFT] + p.ep.off_ret) +
                              static_cast<long long>(tag & EP_TAG_MASK) * p.ldc;
                else
                  atomicCAS(p.ep.status, 0, 3);
              }
            } else {
              rowptr[j] = reinterpret_cast<__nv_bfloat16*>(cbase) + static_cast<long long>(g) * p.c_group_stride +
                          static_cast<long long>(rr) * p.ldc;
            }
          }
          if (p.ep.scat_on && p.ep.row_val && nt == 0 && col_half == 0 && row_ok) {
            const int tag = __ldcg(p.ep.row_tag + row);
            if (tag >= 0 && (tag >> EP_TAG_SHIFT) < p.ep.W && (tag & EP_TAG_MASK) < p.ep.ret_rows)
              reinterpret_cast<float*>(p.ep.peers.base[tag >> EP_TAG_SHIFT] + p.ep.off_ret_vals)[tag & EP_TAG_MASK] =
                  p.ep.row_val[row];
          }
        }
        constexpr int CH = BN / 32 / (EPI_WARPS / 4);
#pragma unroll 1
        for (int c = col_half * CH; c < (col_half + 1) * CH; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;  // uniform across the warp
          uint32_t v[32];
          if (nkb > 0) {
            tmem_ld_32x32b_x32(t_row + c * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          const bool full_chunk = (col0 + 32 <= p.N);
          if (full_chunk) {
            // warp-uniform branch: every lane takes part in the transposition, rows past M are skipped on the way out
            const uint32_t st = smem_u32(epi_stage + (warp - 2) * L::EPI_STAGE_BYTES);
            __syncwarp();  // the previous chunk's readers are done with the staging area
#pragma unroll
            for (int i = 0; i < 8; ++i)
              st_shared_v4(epi_piece_addr(st, lane, i), v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            __syncwarp();
            const int row_base = mt * BM + lane_group * 32;
            const long long gbase = static_cast<long long>(g) * p.c_group_stride;
            if (p.c_fp32) {
              const int q = lane & 7;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int r = (lane >> 3) + 4 * j;
                if (row_base + r >= p.M) continue;
                uint32_t w0, w1, w2, w3;
                ld_shared_v4(epi_piece_addr(st, r, q), w0, w1, w2, w3);
                float4 o = make_float4(__uint_as_float(w0), __uint_as_float(w1), __uint_as_float(w2), __uint_as_float(w3));
                float* dst = reinterpret_cast<float*>(cbase) + gbase + static_cast<long long>(row_base + r) * p.ldc + col0 + 4 * q;
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(dst);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst) = o;
              }
            } else {
              const int q = lane & 3;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int r = (lane >> 2) + 8 * j;
                if (rowptr[j] == nullptr) continue;
                uint32_t w[8];
                ld_shared_v4(epi_piece_addr(st, r, 2 * q), w[0], w[1], w[2], w[3]);
                ld_shared_v4(epi_piece_addr(st, r, 2 * q + 1), w[4], w[5], w[6], w[7]);
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(w[e]);
                __nv_bfloat16* dst = rowptr[j] + col0 + 8 * q;
                if (p.residual) {
                  const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(row_base + r) * p.ldr + col0 + 8 * q);
                  const float2 a = unpack_bf16(rr.x), b = unpack_bf16(rr.y), c2 = unpack_bf16(rr.z), d = unpack_bf16(rr.w);
                  f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y; f[4] += c2.x; f[5] += c2.y; f[6] += d.x; f[7] += d.y;
                }
                if (p.accumulate) {
                  const uint4 rr = *reinterpret_cast<const uint4*>(dst);
                  const float2 a = unpack_bf16(rr.x), b = unpack_bf16(rr.y), c2 = unpack_bf16(rr.z), d = unpack_bf16(rr.w);
                  f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y; f[4] += c2.x; f[5] += c2.y; f[6] += d.x; f[7] += d.y;
                }
                uint4 o;
                o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
                o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
                *reinterpret_cast<uint4*>(dst) = o;
              }
            }
            continue;
          }
          if (!row_ok) continue;
          if (p.c_fp32) {
            float* dst = reinterpret_cast<float*>(cbase) + coff + col0;
            if (full_chunk) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 o = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]),
                                       __uint_as_float(v[i + 3]));
                if (p.accumulate) {
                  float4 old = *reinterpret_cast<float4*>(dst + i);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst + i) = o;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {  // constant indices keep v[] in registers
                if (col0 + i < p.N) {
                  float o = __uint_as_float(v[i]);
                  if (p.accumulate) o += dst[i];
                  dst[i] = o;
                }
              }
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(cbase) + coff + col0;
            const __nv_bfloat16* res = p.residual ? p.residual + static_cast<long long>(row) * p.ldr + col0 : nullptr;
            if (full_chunk) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[i + j]);
                if (res) {
                  uint4 r = *reinterpret_cast<const uint4*>(res + i);
                  float2 a = unpack_bf16(r.x), b = unpack_bf16(r.y), c2 = unpack_bf16(r.z), d = unpack_bf16(r.w);
                  f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y;
                  f[4] += c2.x; f[5] += c2.y; f[6] += d.x; f[7] += d.y;
                }
                if (p.accumulate) {
                  uint4 r = *reinterpret_cast<const uint4*>(dst + i);
                  float2 a = unpack_bf16(r.x), b = unpack_bf16(r.y), c2 = unpack_bf16(r.z), d = unpack_bf16(r.w);
                  f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y;
                  f[4] += c2.x; f[5] += c2.y; f[6] += d.x; f[7] += d.y;
                }
                uint4 o;
                o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
                o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
                *reinterpret_cast<uint4*>(dst + i) = o;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (col0 + i < p.N) {
                  float o = __uint_as_float(v[i]);
                  if (res) o += __bfloat162float(res[i]);
                  if (p.accumulate) o += __bfloat162float(dst[i]);
                  dst[i] = __float2bfloat16(o);
                }
              }
            }
          }
        }
      } else {
        // SwiGLU: accumulator columns [0,BN/2) = gate, [BN/2,BN) = up, for output columns n0..n0+BN/2.
        constexpr int HALF = BN / 2;
        const int n0 = nt * HALF;
        const float scale = (p.row_scale && row_ok) ? __ldcg(p.row_scale + row) : 1.0f;
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc;
        __nv_bfloat16* pre = p.preact ? p.preact + static_cast<long long>(row) * p.ld_preact : nullptr;
        constexpr int CH = HALF / 32 / (EPI_WARPS / 4);
#pragma unroll 1
        for (int c = col_half * CH; c < (col_half + 1) * CH; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;
          uint32_t gv[32], uv[32];
          tmem_ld_32x32b_x32(t_row + c * 32, gv);
          tmem_ld_32x32b_x32(t_row + HALF + c * 32, uv);
          tmem_ld_wait();
          const int lim = min(32, p.N - col0);
          if (lim == 32) {
            // all lanes take part (warp-uniform branch): results are packed to bf16, transposed through the staging
            // area in two rounds (out + gate, then up) and stored as 64-byte row segments, 8 rows per instruction
            uint32_t o[16], pg[16], pu[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              // pre-activations are rounded to bf16 first so forward and backward see the same values
              float g0 = __bfloat162float(__float2bfloat16(__uint_as_float(gv[j])));
              float g1 = __bfloat162float(__float2bfloat16(__uint_as_float(gv[j + 1])));
              float u0 = __bfloat162float(__float2bfloat16(__uint_as_float(uv[j])));
              float u1 = __bfloat162float(__float2bfloat16(__uint_as_float(uv[j + 1])));
              float a0 = g0 / (1.0f + __expf(-g0)) * u0 * scale;
              float a1 = g1 / (1.0f + __expf(-g1)) * u1 * scale;
              o[j / 2] = pack_bf16(a0, a1);
              pg[j / 2] = pack_bf16(g0, g1);
              pu[j / 2] = pack_bf16(u0, u1);
            }
            const uint32_t st = smem_u32(epi_stage + (warp - 2) * L::EPI_STAGE_BYTES);
            const int row_base = mt * BM + lane_group * 32;
            const int q = lane & 3;
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              st_shared_v4(epi_piece_addr64(st, lane, i), o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
              if (pre) st_shared_v4(epi_piece_addr64(st + 2048, lane, i), pg[4 * i], pg[4 * i + 1], pg[4 * i + 2], pg[4 * i + 3]);
            }
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int r = (lane >> 2) + 8 * j;
              if (row_base + r >= p.M) continue;
              uint4 w;
              ld_shared_v4(epi_piece_addr64(st, r, q), w.x, w.y, w.z, w.w);
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row_base + r) * p.ldc + col0 + 8 * q) = w;
              if (pre) {
                ld_shared_v4(epi_piece_addr64(st + 2048, r, q), w.x, w.y, w.z, w.w);
                *reinterpret_cast<uint4*>(p.preact + static_cast<long long>(row_base + r) * p.ld_preact + col0 + 8 * q) = w;
              }
            }
            if (pre) {
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; ++i)
                st_shared_v4(epi_piece_addr64(st, lane, i), pu[4 * i], pu[4 * i + 1], pu[4 * i + 2], pu[4 * i + 3]);
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int r = (lane >> 2) + 8 * j;
                if (row_base + r >= p.M) continue;
                uint4 w;
                ld_shared_v4(epi_piece_addr64(st, r, q), w.x, w.y, w.z, w.w);
                *reinterpret_cast<uint4*>(p.preact + static_cast<long long>(row_base + r) * p.ld_preact + p.F + col0 + 8 * q) = w;
              }
            }
            continue;
          }
          if (!row_ok) continue;
          {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (i < lim) {
                float g0 = __bfloat162float(__float2bfloat16(__uint_as_float(gv[i])));
                float u0 = __bfloat162float(__float2bfloat16(__uint_as_float(uv[i])));
                out[col0 + i] = __float2bfloat16(g0 / (1.0f + __expf(-g0)) * u0 * scale);
                if (pre) {
                  pre[col0 + i] = __float2bfloat16(g0);
                  pre[p.F + col0 + i] = __float2bfloat16(u0);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (p.ep.scat_on) __threadfence_system();   // this thread's peer stores are ordered before the "returned" flag
  } else if (p.ep.push_on) {
    // ------------------------------------------------------------ push warps (warps 10..11)
    // Entries are walked in send order (local expert major, owners rotated so that every owner receives from one
    // source at a time).  A warp copies PUSH_CHUNK rows, fences at system scope, then counts the rows per expert:
    // the warp whose count completes an expert raises this rank's flag for that expert on the owner.
    const EpFuse& ep = p.ep;
    const int E = ep.El * ep.W;
    const int vec = ep.H / 8;
    const bool healthy = *reinterpret_cast<volatile int*>(ep.status) == 0;
    auto flag_of = [&](int e) -> int* {
      const int o = e / ep.El;
      return reinterpret_cast<int*>(ep.peers.base[o] + ep.off_flags) + (e - o * ep.El) * ep.W + ep.rank;
    };
    if (healthy) {
      // Chunks are claimed from a counter (sent[E]) instead of being dealt out by CTA index: the owners' tiles wait for
      // rows, so every row must go out even when some CTAs of this grid are not resident yet (another kernel holds
      // their SM).  With a static split the rows of a waiting CTA would never leave while the resident CTAs spin.
      int* next_chunk = ep.sent + E;
      for (;;) {
        long long chunk = 0;
        if (lane == 0) chunk = atomicAdd(next_chunk, 1);
        chunk = __shfl_sync(0xffffffffu, chunk, 0);
        if (chunk == 0) {
          // experts this rank sends nothing to: their owners must not wait for it
          for (int e = lane; e < E; e += 32)
            if (ep.counts[e] == 0) st_release_sys(flag_of(e), ep.epoch);
        }
        const long long c0 = chunk * PUSH_CHUNK;
        if (c0 >= ep.n_entries) break;
        const int cnt = static_cast<int>(ep.n_entries - c0 < PUSH_CHUNK ? ep.n_entries - c0 : PUSH_CHUNK);
        int n_l = -1, e_l = -1, r_l = -1;
        if (lane < cnt) {
          n_l = ep.order[c0 + lane];
          if (n_l >= 0 && n_l < ep.n_entries) {   // a broken order table must not become a wild read
            e_l = ep.expert[n_l];
            r_l = ep.dest_row[n_l];
          }
        }
        for (int j = 0; j < cnt; ++j) {
          const int n = __shfl_sync(0xffffffffu, n_l, j);
          const int e = __shfl_sync(0xffffffffu, e_l, j);
          const int r = __shfl_sync(0xffffffffu, r_l, j);
          const int o = (e >= 0 && e < E) ? e / ep.El : -1;
          if (o < 0 || r < 0 || r >= ep.cap_rows) {   // never write outside the owner's buffer
            if (lane == 0) atomicExch(ep.status, 3);
            continue;
          }
          const uint4* srow = reinterpret_cast<const uint4*>(ep.src + static_cast<long long>(n / ep.k) * ep.lds);
          uint4* drow = reinterpret_cast<uint4*>(ep.peers.base[o] + ep.off_rows) + static_cast<long long>(r) * vec;
          for (int c = lane; c < vec; c += 32 * 8) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (c + 32 * u < vec) v[u] = srow[c + 32 * u];
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (c + 32 * u < vec) drow[c + 32 * u] = v[u];
          }
          if (lane == 0) {
            if (ep.val) reinterpret_cast<float*>(ep.peers.base[o] + ep.off_vals)[r] = ep.val[n];
            reinterpret_cast<int*>(ep.peers.base[o] + ep.off_tags)[r] = (ep.rank << EP_TAG_SHIFT) | n;
          }
        }
        __threadfence_system();
        __syncwarp();
        if (lane < cnt && e_l >= 0 && e_l < E) {
          const int before = atomicAdd(ep.sent + e_l, 1);
          if (before + 1 == ep.counts[e_l]) {
            __threadfence_system();
            st_release_sys(flag_of(e_l), ep.epoch);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
  if (p.ep.scat_on) {
    // the last CTA to get here tells every peer that this rank has returned all of its rows
    if (threadIdx.x == 0) {
      __threadfence_system();
      s_last_cta = (atomicAdd(p.ep.done_counter, 1u) == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last_cta) {
      if (static_cast<int>(threadIdx.x) < p.ep.W) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<int*>(p.ep.peers.base[threadIdx.x] + p.ep.off_ret_flags) + p.ep.rank, p.ep.ret_epoch);
      }
      if (threadIdx.x == 0) *p.ep.done_counter = 0;
    }
  }
}

// ----------------------------------------------------------------------------
// Host launcher
// ----------------------------------------------------------------------------
struct GemmArgs {
  const void* A;      // bf16
  long long lda;      // elements: row stride of A's memory matrix
  const void* B;      // bf16
  long long ldb;      // elements: row stride of B's memory matrix
  long long b_group_stride;  // elements between B[g] (grouped-M), 0 otherwise
  int b_groups;       // number of B groups (>=1)
  void* C;
  long long ldc;
  long long c_group_stride;
  int M, N, K;        // grouped-K: K ignored, M = rows of A^T ( = columns of A memory ), N = cols of B memory
  int a_mn, b_mn;     // memory orientation: 0 = K contiguous, 1 = M/N contiguous
  int c_fp32, accumulate;
  const void* residual;
  long long ldr;
  const int* tile_group;
  int m_tiles_cap;    // grouped-M: number of m tiles to schedule (capacity)
  const int* group_rows;
  int groups_k;
  long long total_rows;  // grouped-K: total rows of A/B memory matrices
  int epi;            // 0 store, 1 swiglu
  int F;
  const float* row_scale;
  void* preact;
  long long ld_preact;
  int num_sms;
  const struct EpFuseArgs* ep;   // optional expert-parallel fusion (grouped-M launches only)
};

// Host description of the expert-parallel fusion of one launch (C ABI; see `EpFuse` for the meaning of the fields).
struct EpFuseArgs {
  const unsigned long long* peer_ptrs;   // [W] base address of every rank's symmetric buffer
  int W, rank, El;
  int* status;
  long long budget_ms;
  // push prologue
  int push_on;
  long long off_rows, off_vals, off_tags, off_flags;
  const void* src;
  long long lds;
  const int* order;
  const int* expert;
  const int* dest_row;
  const float* val;
  const int* counts;
  int* sent;
  int n_entries, k, H, epoch;
  long long cap_rows;
  // scatter epilogue
  int scat_on;
  long long off_ret, off_ret_vals, off_ret_flags;
  const int* row_tag;
  const float* row_val;
  int ret_epoch;
  unsigned int* done_counter;
  int ret_rows;
};

template <int BN, bool A_MN, bool B_MN, int EPI>
static int launch(const GemmArgs& a, cudaStream_t stream) {
  using L = SmemLayout<BN, A_MN, B_MN>;
  CUtensorMap tmA, tmB;
  // ---- A map (2D)
  {
    uint64_t dims[2];
    uint64_t str[1] = {static_cast<uint64_t>(a.lda) * 2};
    uint32_t box[2];
    if (!A_MN) {
      // memory [M rows][K contiguous]
      dims[0] = static_cast<uint64_t>(a.K);
      dims[1] = static_cast<uint64_t>(a.M);
      box[0] = BK;
      box[1] = BM;
    } else {
      // memory [K rows][M contiguous]
      dims[0] = static_cast<uint64_t>(a.M);
      dims[1] = static_cast<uint64_t>(a.groups_k > 0 ? a.total_rows : a.K);
      box[0] = 64;
      box[1] = BK;
    }
    int r = make_tmap_bf16(&tmA, a.A, 2, dims, str, box);
    if (r) return 10000 + r;
  }
  // ---- B map (3D, last dim = group)
  const int n_mem = (EPI == EPI_SWIGLU) ? 2 * a.F : a.N;
  {
    uint64_t dims[3];
    uint64_t str[2];
    uint32_t box[3];
    str[0] = static_cast<uint64_t>(a.ldb) * 2;
    const uint64_t rows_b = !B_MN ? static_cast<uint64_t>(n_mem)
                                  : static_cast<uint64_t>(a.groups_k > 0 ? a.total_rows : a.K);
    str[1] = a.b_groups > 1 ? static_cast<uint64_t>(a.b_group_stride) * 2 : rows_b * str[0];
    dims[2] = static_cast<uint64_t>(a.b_groups > 1 ? a.b_groups : 1);
    if (!B_MN) {
      // memory [N rows][K contiguous]
      dims[0] = static_cast<uint64_t>(a.K);
      dims[1] = rows_b;
      box[0] = BK;
      box[1] = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
    } else {
      // memory [K rows][N contiguous]
      dims[0] = static_cast<uint64_t>(n_mem);
      dims[1] = rows_b;
      box[0] = 64;
      box[1] = BK;
    }
    box[2] = 1;
    int r = make_tmap_bf16(&tmB, a.B, 3, dims, str, box);
    if (r) return 20000 + r;
  }
  GemmParams p;
  memset(&p.ep, 0, sizeof(p.ep));
  if (a.ep) {
    const EpFuseArgs& e = *a.ep;
    for (int i = 0; i < MAX_RANKS; ++i) p.ep.peers.base[i] = i < e.W ? e.peer_ptrs[i] : 0ull;
    p.ep.W = e.W; p.ep.rank = e.rank; p.ep.El = e.El; p.ep.status = e.status;
    p.ep.budget_ns = static_cast<unsigned long long>(e.budget_ms) * 1000000ull;
    p.ep.push_on = e.push_on;
    p.ep.off_rows = e.off_rows; p.ep.off_vals = e.off_vals; p.ep.off_tags = e.off_tags; p.ep.off_flags = e.off_flags;
    p.ep.src = reinterpret_cast<const __nv_bfloat16*>(e.src); p.ep.lds = e.lds;
    p.ep.order = e.order; p.ep.expert = e.expert; p.ep.dest_row = e.dest_row; p.ep.val = e.val;
    p.ep.counts = e.counts; p.ep.sent = e.sent;
    p.ep.n_entries = e.n_entries; p.ep.k = e.k; p.ep.H = e.H; p.ep.epoch = e.epoch; p.ep.cap_rows = e.cap_rows;
    p.ep.scat_on = e.scat_on;
    p.ep.off_ret = e.off_ret; p.ep.off_ret_vals = e.off_ret_vals; p.ep.off_ret_flags = e.off_ret_flags;
    p.ep.row_tag = e.row_tag; p.ep.row_val = e.row_val; p.ep.ret_epoch = e.ret_epoch;
    p.ep.done_counter = e.done_counter;
    p.ep.ret_rows = e.ret_rows;
  }
  p.M = a.M; p.N = a.N; p.K = a.K;
  constexpr int TN = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  p.m_tiles = a.tile_group ? a.m_tiles_cap : (a.M + BM - 1) / BM;
  p.n_tiles = (a.N + TN - 1) / TN;
  p.groups_k = a.groups_k;
  p.C = a.C; p.ldc = a.ldc; p.c_group_stride = a.c_group_stride;
  p.c_fp32 = a.c_fp32; p.accumulate = a.accumulate;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual); p.ldr = a.ldr;
  p.tile_group = a.tile_group; p.group_rows = a.group_rows;
  p.F = a.F; p.row_scale = a.row_scale;
  p.preact = reinterpret_cast<__nv_bfloat16*>(a.preact); p.ld_preact = a.ld_preact;

  auto kfn = gemm_kernel<BN, A_MN, B_MN, EPI>;
  static bool smem_done[16] = {};
  {
    const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kfn), L::TOTAL, smem_done);
    if (e != cudaSuccess) return 300 + static_cast<int>(e);
  }
  long long total = static_cast<long long>(p.m_tiles) * p.n_tiles * (p.groups_k > 0 ? p.groups_k : 1);
  if (total <= 0) return 0;
  int grid = static_cast<int>(total < a.num_sms ? total : a.num_sms);
  kfn<<<grid, p.ep.push_on ? GEMM_THREADS_PUSH : GEMM_THREADS, L::TOTAL, stream>>>(tmA, tmB, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + static_cast<int>(e);
}

}  // namespace ttb

// Returns 0 on success; non-zero codes: 10000+r / 20000+r tensor-map encode failure of A / B (r = CUresult),
// 300+e shared-memory opt-in, 400+e launch (e = cudaError_t), 9xx bad arguments.
TTB_EXPORT int ttb_gemm_bf16(const ttb::GemmArgs* args, void* stream_ptr) {
  using namespace ttb;
  const GemmArgs& a = *args;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  if ((a.lda % 8) || (a.ldb % 8)) return 901;
  if ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.B)) & 15) return 902;
  // vectorised epilogue stores: 16-byte aligned rows
  if (a.c_fp32 ? (a.ldc % 4) : (a.ldc % 8)) return 903;
  if (reinterpret_cast<uintptr_t>(a.C) & 15) return 903;
  if (a.residual && ((a.ldr % 8) || (reinterpret_cast<uintptr_t>(a.residual) & 15))) return 904;
  if (a.epi == EPI_SWIGLU && ((a.F % 8) || a.c_fp32 || (a.preact && (a.ld_preact % 8)))) return 905;
  if (a.ep) {
    const EpFuseArgs& e = *a.ep;
    if (!a.tile_group || a.groups_k > 0 || e.W < 1 || e.W > MAX_RANKS || e.El < 1 || e.El * e.W > 1024 || !e.status) return 906;
    if (e.push_on && (a.a_mn || (e.H % 8) || (e.lds % 8) || !e.order || !e.expert || !e.dest_row || !e.counts || !e.sent ||
                      e.n_entries < 0 || e.n_entries > EP_TAG_MASK || (e.off_rows % 16)))
      return 907;
    // the scatter epilogue lives in the bf16 row-major store path: whole 32-column chunks, no residual / accumulate
    if (e.scat_on && (a.epi != EPI_STORE || a.c_fp32 || a.accumulate || a.residual || (a.N % 32) || !e.row_tag ||
                      !e.done_counter || (e.off_ret % 16)))
      return 908;
  }
  const bool wide = (a.epi == EPI_SWIGLU) ? true : (a.N > 128);
#define TTB_DISPATCH(AMN, BMN)                                                             \
  if (a.epi == EPI_SWIGLU) return launch<256, AMN, BMN, EPI_SWIGLU>(a, stream);            \
  if (wide) return launch<256, AMN, BMN, EPI_STORE>(a, stream);                            \
  return launch<128, AMN, BMN, EPI_STORE>(a, stream);
  if (!a.a_mn && !a.b_mn) { TTB_DISPATCH(false, false) }
  if (!a.a_mn && a.b_mn) { TTB_DISPATCH(false, true) }
  if (a.a_mn && a.b_mn) { TTB_DISPATCH(true, true) }
  if (a.a_mn && !a.b_mn) { TTB_DISPATCH(true, false) }
#undef TTB_DISPATCH
  return 999;
}

TTB_EXPORT int ttb_gemm_status(unsigned int* out4, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out4, ttb::g_status_word, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (reset) {
    unsigned int z[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(ttb::g_status_word, z, sizeof(z));
  }
  return static_cast<int>(e);
}
