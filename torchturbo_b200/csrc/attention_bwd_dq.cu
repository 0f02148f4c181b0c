// Query-gradient pass of the variable-length flash attention backward for sm_100a: dQ without atomics.
//
// One CTA owns one 128-row query tile of one document for one query head and walks the KV blocks that the tile can
// see, as the forward kernel does; per block, all on tcgen05 with M = 128:
//     S  = Q_i K_j^T            [q, kv]   (K-major x K-major)
//     dP = dO_i V_j^T           [q, kv]   (K-major x K-major)
//     P  = exp2(S c - lse_q),   dS = P (dP - Delta_q) scale     (thread = query row; bf16 pairs written to TMEM)
//     dQ += dS K_j              [q, d]    (A from TMEM, K_j MN-major straight from its [kv, d] tile)
// dQ accumulates in TMEM over the whole tile and is written once, so the result does not depend on the order in which
// CTAs finish: this pass is the bit-reproducible alternative to the atomically reduced dQ of `attn_bwd_kernel`, and
// the only dQ path for query / key heads 192 wide (multi-head latent attention), whose dQ^T, dK and dV accumulators
// do not fit tensor memory together.  It recomputes S and dP (7 products per tile pair over both passes instead of 5).
// Warp roles: 0 TMA producer (Q and dO once, K_j in two stages, V_j in two stages or one for 192-wide heads),
// 1 MMA issuer, 2-9 softmax (warps 2-5 take kv columns 0-63 of the block, warps 6-9 columns 64-127).  Every wait is
// bounded; on a timeout the roles drain to the final barrier, TMEM is freed and the status word records kernel / site.
//
// Counterpart of flash-attn 2's backward used through the reference attention interface
// (models/modules/attention/interface.py:114-158), which offers a deterministic mode as well.
#include "common.cuh"

namespace ttb {

constexpr unsigned KID_ATTN_DQ = 5;
constexpr int DQ_TILE = 128 * 128 * 2;   // a [128 x 128] bf16 tile

struct AttnDqParams {
  const int* q_tiles;   // [n_tiles, 3]: first query row, document start, document end
  const float* lse;     // [Hq, T]
  const float* delta;   // [Hq, T]
  __nv_bfloat16* dq;    // [T, Hq, DQK]
  int Hq, Hk;
  long long T;
  float scale;
  int causal;
};

template <int DQK>
struct DqSmem {
  static constexpr int QK_BYTES = 128 * DQK * 2;
  static constexpr int VS = DQK == 128 ? 2 : 1;          // V stages
  static constexpr int Q = 0;
  static constexpr int DO = Q + QK_BYTES;
  static constexpr int K0 = DO + DQ_TILE;
  static constexpr int V0 = K0 + 2 * QK_BYTES;
  static constexpr int BARS = V0 + VS * DQ_TILE;
  static constexpr int TOTAL = BARS + 256 + 1024;
};

__device__ __forceinline__ float dq_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int DQK>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const AttnDqParams p) {
  using Smem = DqSmem<DQK>;
  constexpr int QK_BYTES = Smem::QK_BYTES, VS = Smem::VS, NP = DQK / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Smem::BARS);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // S and dP of a block are in TMEM
  uint64_t* s_empty = bars + 10;  // every softmax warp has its copy
  uint64_t* ds_full = bars + 11;  // dS of a block is in TMEM
  uint64_t* ds_empty = bars + 12; // dS K of a block retired
  uint64_t* dq_done = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.y, h = blockIdx.x;     // heads vary fastest: the longest tiles of all heads start first
  const int hk = h / (p.Hq / p.Hk);
  const int q0 = p.q_tiles[tile * 3 + 0];
  const int ds = p.q_tiles[tile * 3 + 1];
  const int de = p.q_tiles[tile * 3 + 2];
  const int kv_end = p.causal ? min(de, q0 + 128) : de;
  const int nblk = (kv_end - ds + 127) / 128;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
    }
    mbar_init(s_full, 1); mbar_init(s_empty, 8);
    mbar_init(ds_full, 8); mbar_init(ds_empty, 1);
    mbar_init(dq_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_S = tmem_base;              // 128 columns
  const uint32_t tm_DP = tmem_base + 128;       // 128 columns
  const uint32_t tm_DQ = tmem_base + 256;       // DQK columns
  const uint32_t tm_DS = tmem_base + 256 + DQK; // 64 columns: bf16 pairs, column = kv index / 2

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmDO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, QK_BYTES + DQ_TILE);
#pragma unroll
      for (int pn = 0; pn < NP; ++pn) tma_load_2d(smem + Smem::Q + pn * 16384, &tmQ, q_full, h * DQK + pn * 64, q0);
      tma_load_2d(smem + Smem::DO, &tmDO, q_full, h * 128, q0);
      tma_load_2d(smem + Smem::DO + 16384, &tmDO, q_full, h * 128 + 64, q0);
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1, vs = j % VS;
        const int kv0 = ds + j * 128;
        if (!mbar_wait(&k_empty[st], ((j >> 1) & 1) ^ 1, KID_ATTN_DQ, 1)) break;
        mbar_expect_tx(&k_full[st], QK_BYTES);
#pragma unroll
        for (int pn = 0; pn < NP; ++pn)
          tma_load_2d(smem + Smem::K0 + st * QK_BYTES + pn * 16384, &tmK, &k_full[st], hk * DQK + pn * 64, kv0);
        if (!mbar_wait(&v_empty[vs], ((j / VS) & 1) ^ 1, KID_ATTN_DQ, 2)) break;
        mbar_expect_tx(&v_full[vs], DQ_TILE);
        tma_load_2d(smem + Smem::V0 + vs * DQ_TILE, &tmV, &v_full[vs], hk * 128, kv0);
        tma_load_2d(smem + Smem::V0 + vs * DQ_TILE + 16384, &tmV, &v_full[vs], hk * 128 + 64, kv0);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t id_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t id_dq = make_idesc_bf16(128, DQK, false, true);
      const uint32_t sQ = smem_u32(smem + Smem::Q), sDO = smem_u32(smem + Smem::DO);
      bool ok = mbar_wait(q_full, 0, KID_ATTN_DQ, 3);
      auto issue_scores = [&](int j) -> bool {
        const int st = j & 1, vs = j % VS;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1, KID_ATTN_DQ, 4)) return false;
        if (!mbar_wait(&v_full[vs], (j / VS) & 1, KID_ATTN_DQ, 5)) return false;
        if (!mbar_wait(s_empty, (j & 1) ^ 1, KID_ATTN_DQ, 6)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + Smem::K0 + st * QK_BYTES);
        const uint32_t sV = smem_u32(smem + Smem::V0 + vs * DQ_TILE);
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_ss(tm_S, make_smem_desc(sQ + off, 16, 1024), make_smem_desc(sK + off, 16, 1024), id_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_ss(tm_DP, make_smem_desc(sDO + off, 16, 1024), make_smem_desc(sV + off, 16, 1024), id_s, kk != 0);
        }
        umma_commit(s_full);
        umma_commit(&v_empty[vs]);
        return true;
      };
      if (ok && nblk > 0) ok = issue_scores(0);
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk && !issue_scores(j + 1)) { ok = false; break; }
        if (!mbar_wait(ds_full, j & 1, KID_ATTN_DQ, 7)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + Smem::K0 + (j & 1) * QK_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A = dS from TMEM (a k-step of 16 kv columns is 8 packed columns); B = K: MN-major [kv rows][d], a k-step of
          // 16 kv rows = 2048 bytes, d panels 16 KB apart
          umma_ts(tm_DQ, tm_DS + kk * 8, make_smem_desc(sK + kk * 2048, 16384, 1024), id_dq, (j | kk) != 0);
        }
        umma_commit(&k_empty[j & 1]);
        umma_commit(ds_empty);
      }
      if (ok) umma_commit(dq_done);
    }
  } else {
    // ---------------------------------------------------------------- softmax / dS (thread = query row, 64 kv columns)
    const int lg = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = lg * 32 + lane;
    const int qrow = q0 + row;
    const bool row_ok = qrow < de;
    const float c = p.scale * 1.4426950408889634f;
    const uint32_t lane_off = static_cast<uint32_t>(lg * 32) << 16;
    const long long stat = static_cast<long long>(h) * p.T + qrow;
    const float neg_lse = row_ok ? -p.lse[stat] * 1.4426950408889634f : -INFINITY;
    const float neg_delta = row_ok ? -p.delta[stat] * p.scale : 0.f;
    const uint64_t cc = f2_pack(c, c), nl = f2_pack(neg_lse, neg_lse);
    const uint64_t sc2 = f2_pack(p.scale, p.scale), nd = f2_pack(neg_delta, neg_delta);
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      if (!mbar_wait(s_full, j & 1, KID_ATTN_DQ, 8)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = ds + j * 128 + half * 64;
      float s[64], dp[64];
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
        uint32_t va[32], vb[32];
        tmem_ld_32x32b_x32(tm_S + half * 64 + cb * 32 + lane_off, va);
        tmem_ld_32x32b_x32(tm_DP + half * 64 + cb * 32 + lane_off, vb);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          s[cb * 32 + i] = __uint_as_float(va[i]);
          dp[cb * 32 + i] = __uint_as_float(vb[i]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty);
      const bool need_mask = (kv0 + 64 > de) || (p.causal && kv0 + 63 > q0);
      const int lim = p.causal ? min(de - 1, qrow) : de - 1;  // last visible kv index
      uint32_t w[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float a0, a1;
        f2_unpack(f2_fma(f2_pack(s[2 * i], s[2 * i + 1]), cc, nl), a0, a1);
        float p0 = dq_exp2(a0), p1 = dq_exp2(a1);
        if (need_mask) {
          p0 = (row_ok && kv0 + 2 * i <= lim) ? p0 : 0.f;
          p1 = (row_ok && kv0 + 2 * i + 1 <= lim) ? p1 : 0.f;
        }
        float d0, d1;
        f2_unpack(f2_mul(f2_pack(p0, p1), f2_fma(f2_pack(dp[2 * i], dp[2 * i + 1]), sc2, nd)), d0, d1);
        w[i] = pack_bf16(d0, d1);
      }
      // the dS buffer was read by the product of the previous block
      if (j > 0) {
        if (!mbar_wait(ds_empty, (j - 1) & 1, KID_ATTN_DQ, 9)) { ok = false; break; }
        tc_fence_after();
      }
      tmem_st_32x32b_x32(tm_DS + half * 32 + lane_off, w);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    // ---- epilogue: each half writes its share of the dQ columns
    if (ok && nblk > 0) ok = mbar_wait(dq_done, 0, KID_ATTN_DQ, 10);
    if (ok) {
      tc_fence_after();
      constexpr int COLS = DQK / 2;               // 64 or 96 columns per half
      __nv_bfloat16* dst = p.dq + (static_cast<long long>(qrow) * p.Hq + h) * DQK + half * COLS;
#pragma unroll
      for (int cb = 0; cb < COLS / 32; ++cb) {
        uint32_t v[32];
        if (nblk > 0) {
          tmem_ld_32x32b_x32(tm_DQ + half * COLS + cb * 32 + lane_off, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
            o.y = pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            o.z = pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
            o.w = pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
            *reinterpret_cast<uint4*>(dst + cb * 32 + i) = o;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static int dq_rows_map(CUtensorMap* m, const void* base, long long rows, long long row_stride_elems, int cols) {
  uint64_t dims[2] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows)};
  uint64_t str[1] = {static_cast<uint64_t>(row_stride_elems) * 2};
  uint32_t box[2] = {64, 128};
  return make_tmap_bf16(m, base, 2, dims, str, box);
}

template <int DQK>
static int launch_attn_dq(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tk, const CUtensorMap& tv,
                          const AttnDqParams& p, int n_tiles, cudaStream_t stream) {
  static bool smem_done[16] = {};
  const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(attn_bwd_dq_kernel<DQK>), DqSmem<DQK>::TOTAL, smem_done);
  if (e != cudaSuccess) return 300 + static_cast<int>(e);
  dim3 grid(p.Hq, n_tiles);
  attn_bwd_dq_kernel<DQK><<<grid, 320, DqSmem<DQK>::TOTAL, stream>>>(tq, tdo, tk, tv, p);
  return 0;
}

}  // namespace ttb

using namespace ttb;

// q: [T, Hq*D] contiguous rows; dout: [T, Hq*128] contiguous; k: [T, Hk*D] (ldk); v: [T, Hk*128] (ldv); lse, delta:
// fp32 [Hq, T] (delta = rowsum(dO * O), from the backward's row-dot kernel); dq: bf16 [T, Hq, D], rows outside every
// document are not written.  D = 128 or 192.
TTB_EXPORT int ttb_attn_bwd_dq(const void* q, const void* k, long long ldk, const void* v, long long ldv, const void* dout,
                               const float* lse, const float* delta, void* dq, const int* q_tiles, int n_tiles, long long T,
                               int Hq, int Hk, int D, float scale, int causal, void* stream_ptr) {
  if ((D != 128 && D != 192) || Hq % Hk) return 901;
  if ((ldk % 8) || (ldv % 8)) return 902;
  if (T == 0 || n_tiles == 0) return 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  CUtensorMap tq, tdo, tk, tv;
  if (dq_rows_map(&tq, q, T, (long long)Hq * D, Hq * D)) return 101;
  if (dq_rows_map(&tdo, dout, T, (long long)Hq * 128, Hq * 128)) return 102;
  if (dq_rows_map(&tk, k, T, ldk, Hk * D)) return 103;
  if (dq_rows_map(&tv, v, T, ldv, Hk * 128)) return 104;
  AttnDqParams p{q_tiles, lse, delta, (__nv_bfloat16*)dq, Hq, Hk, T, scale, causal};
  const int rc = D == 128 ? launch_attn_dq<128>(tq, tdo, tk, tv, p, n_tiles, stream)
                          : launch_attn_dq<192>(tq, tdo, tk, tv, p, n_tiles, stream);
  if (rc) return rc;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
