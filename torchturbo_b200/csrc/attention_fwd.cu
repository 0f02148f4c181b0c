// Variable-length (packed) flash attention forward for sm_100a, GQA, causal or full; value heads 128 wide, query / key
// heads 128 wide or 192 (multi-head latent attention: 128 without position + 64 rotary).
//
// One CTA handles one 128-row query tile of one document for one query head.  Warp roles:
//   warp 0      TMA producer   : Q once, then K_j (3 stages) / V_j (2 stages) tiles
//   warp 1      MMA issuer     : S_j = Q K_j^T  (tcgen05, fp32 in TMEM, 2 buffers)
//                                O  += P_j V_j  (P read from TMEM, V MN-major straight from its [kv, d] tile; O stays
//                                               in TMEM)
//   warps 2-9   softmax        : thread = query row; warps 2-5 take kv columns 0-63 of the block, warps 6-9 columns
//                                64-127 (a warp may read the TMEM lanes 32 (warp % 4) .. +31 at any column), so the
//                                dependent chain per block is half as long.  The halves exchange their row maxima
//                                through shared memory, write P_j as packed bf16 pairs into TMEM (two buffers: the
//                                A operand of P.V comes from tensor memory, which spares the shared-memory
//                                bandwidth that the K / V operands and the TMA writes already use up) and keep
//                                partial row sums.
// The output accumulator is never copied out between blocks.  The running maximum of a row is raised only when the
// new block exceeds it by more than 2^8 in the exponent (probabilities then stay below 256, exact in fp32 sums and
// harmless in bf16); only then the row's accumulator is rescaled in place (tcgen05.ld / multiply / tcgen05.st by the
// softmax warps, each half its 64 output columns) before the block's P.V is issued.  The normalisation by the row
// sum at the end uses the same maximum, so the result does not depend on when the maximum was raised.
// Every wait is bounded (mbar_wait): on timeout the role stops, all roles meet at the final barrier,
// TMEM is released and the status word records kernel/site.
//
// Replaces flash-attn 2 `flash_attn_varlen_func` used by the reference (models/modules/attention/interface.py:114-158)
// and produces the optional per-head maximum logit of its TE / FlexAttention providers
// (ops/providers/cuda/attention.py:34-331).
#include "common.cuh"

namespace ttb {

constexpr unsigned KID_ATTN_FWD = 2;
constexpr int AT_BM = 128;   // query rows per CTA
constexpr int AT_BN = 128;   // kv rows per block
constexpr int AT_D = 128;    // head dim
constexpr int TILE_BYTES = 128 * 128 * 2;  // one [128 x 128] bf16 tile = two 16 KB swizzle panels
constexpr float AT_LAZY = 8.f;             // raise the running maximum only beyond this many powers of two

struct AttnFwdParams {
  const int* q_tiles;   // [n_tiles, 3]: first query row, document start, document end (token indices)
  __nv_bfloat16* out;   // [T, Hq, D]
  float* lse;           // [Hq, T] natural-log logsumexp of the scaled logits (or null)
  float* max_logit;     // [Hq] per-head maximum scaled logit (atomic max; or null)
  int Hq, Hk;
  long long T;
  float scale;          // softmax scale (1/sqrt(D))
  int causal;
};

template <int DQK>
struct AttnSmem {
  // tiles of 128 rows in 64-column swizzle panels of 16 KB, 1024-byte aligned
  static constexpr int QK_BYTES = 128 * DQK * 2;          // one Q or K tile
  static constexpr int KS = DQK == 128 ? 3 : 2;           // K stages
  static constexpr int Q = 0;
  static constexpr int K0 = Q + QK_BYTES;
  static constexpr int V0 = K0 + KS * QK_BYTES;
  static constexpr int ROWMAX = V0 + 2 * TILE_BYTES;      // float [2 parities][2 halves][128]
  static constexpr int ROWSUM = ROWMAX + 4 * 128 * 4;     // float [2 halves][128]
  static constexpr int BARS = ROWSUM + 2 * 128 * 4;
  static constexpr int TOTAL = BARS + 256 + 1024;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
  // valid for any sign mix: compare as ordered ints
  if (v >= 0.f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

template <int DQK>
__global__ void __launch_bounds__(320, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using AttnSmem = ttb::AttnSmem<DQK>;
  constexpr int KS = AttnSmem::KS, QK_BYTES = AttnSmem::QK_BYTES, NP = DQK / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttnSmem::BARS);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [3]
  uint64_t* k_empty = bars + 4;   // [3]
  uint64_t* v_full = bars + 7;    // [2]
  uint64_t* v_empty = bars + 9;   // [2]
  uint64_t* s_full = bars + 11;   // [2]
  uint64_t* s_empty = bars + 13;  // [2]
  uint64_t* p_full = bars + 15;
  uint64_t* p_empty = bars + 16;  // [2] P_j V_j retired: that P buffer may be rewritten, O holds blocks 0..j
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* s_dead = reinterpret_cast<volatile int*>(bars + 19);   // a softmax warp's wait gave up
  float* s_rowmax = reinterpret_cast<float*>(smem + AttnSmem::ROWMAX);
  float* s_rowsum = reinterpret_cast<float*>(smem + AttnSmem::ROWSUM);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads vary fastest in launch order: the tile table lists the tiles with the most KV blocks first, so every head's
  // longest tiles start before any short one, and neighbouring CTAs (the query heads of a group) read the same K / V
  const int tile = blockIdx.y, h = blockIdx.x;
  const int hk = h / (p.Hq / p.Hk);
  const int q0 = p.q_tiles[tile * 3 + 0];
  const int ds = p.q_tiles[tile * 3 + 1];
  const int de = p.q_tiles[tile * 3 + 2];
  const int kv_end = p.causal ? min(de, q0 + AT_BM) : de;
  const int nblk = (kv_end - ds + AT_BN - 1) / AT_BN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 8);
    }
    mbar_init(p_full, 8);
    mbar_init(&p_empty[0], 1);
    mbar_init(&p_empty[1], 1);
    *s_dead = 0;
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
  const uint32_t tm_S = tmem_base;        // 2 x 128 columns
  const uint32_t tm_O = tmem_base + 256;  // 128 columns
  const uint32_t tm_P = tmem_base + 384;  // 2 x 64 columns: bf16 pairs, column = kv index / 2

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, QK_BYTES);
#pragma unroll
      for (int pn = 0; pn < NP; ++pn) tma_load_2d(smem + AttnSmem::Q + pn * 16384, &tmQ, q_full, h * DQK + pn * 64, q0);
      bool ok = true;
      auto load_k = [&](int j) -> bool {
        const int ks = j % KS;
        if (!mbar_wait(&k_empty[ks], ((j / KS) & 1) ^ 1, KID_ATTN_FWD, 1)) return false;
        const int kv0 = ds + j * AT_BN;
        mbar_expect_tx(&k_full[ks], QK_BYTES);
#pragma unroll
        for (int pn = 0; pn < NP; ++pn)
          tma_load_2d(smem + AttnSmem::K0 + ks * QK_BYTES + pn * 16384, &tmK, &k_full[ks], hk * DQK + pn * 64, kv0);
        return true;
      };
      // K runs one block ahead of V, so that a wait for a V buffer never holds back the next K request
      if (nblk > 0) ok = load_k(0);
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk && !load_k(j + 1)) { ok = false; break; }
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int kv0 = ds + j * AT_BN;
        if (!mbar_wait(&v_empty[st], ph ^ 1, KID_ATTN_FWD, 2)) { ok = false; break; }
        mbar_expect_tx(&v_full[st], TILE_BYTES);
        tma_load_2d(smem + AttnSmem::V0 + st * TILE_BYTES, &tmV, &v_full[st], hk * AT_D, kv0);
        tma_load_2d(smem + AttnSmem::V0 + st * TILE_BYTES + 16384, &tmV, &v_full[st], hk * AT_D + 64, kv0);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);  // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);   // P (K-major) x V (MN-major)
      const uint32_t sQ = smem_u32(smem + AttnSmem::Q);
      bool ok = mbar_wait(q_full, 0, KID_ATTN_FWD, 3);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int ks = j % KS;
        if (!mbar_wait(&k_full[ks], (j / KS) & 1, KID_ATTN_FWD, 4)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, KID_ATTN_FWD, 5)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + AttnSmem::K0 + ks * QK_BYTES);
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_ss(tm_S + st * 128, make_smem_desc(sQ + off, 16, 1024), make_smem_desc(sK + off, 16, 1024), idesc_s,
                  kk != 0);
        }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[ks]);
        return true;
      };
      if (ok && nblk > 0) ok = issue_s(0);
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          if (!issue_s(j + 1)) { ok = false; break; }
        }
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&v_full[st], ph, KID_ATTN_FWD, 6)) { ok = false; break; }
        // P_j written and, where a row maximum was raised, O rescaled in place
        if (!mbar_wait(p_full, j & 1, KID_ATTN_FWD, 7)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sV = smem_u32(smem + AttnSmem::V0 + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A = P from TMEM: a k-step of 16 kv columns is 8 packed columns
          // B = V: MN-major [kv rows][d], k-step of 16 kv rows = 2048 bytes, d panels 16 KB apart
          umma_ts(tm_O, tm_P + st * 64 + kk * 8, make_smem_desc(sV + kk * 2048, 16384, 1024), idesc_o, (j | kk) != 0);
        }
        umma_commit(&v_empty[st]);
        umma_commit(&p_empty[st]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax (thread = query row, 64 kv columns)
    const int lg = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = lg * 32 + lane;
    const int qrow = q0 + row;
    const bool row_ok = qrow < de;
    const float c = p.scale * 1.4426950408889634f;
    const uint32_t lane_off = static_cast<uint32_t>(lg * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f, mx_logit = -INFINITY;
    bool ok = true;
    // one kv block; false when a wait gave up
    auto block = [&](int j, float (&s)[64], float& m_half) -> bool {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[st], ph, KID_ATTN_FWD, 9)) return false;
      tc_fence_after();
      const int kv0 = ds + j * AT_BN + half * 64;
      const uint32_t t_row = tm_S + st * 128 + half * 64 + lane_off;
      {
        uint32_t va[32], vb[32];
        tmem_ld_32x32b_x32(t_row, va);
        tmem_ld_32x32b_x32(t_row + 32, vb);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          s[i] = __uint_as_float(va[i]);
          s[32 + i] = __uint_as_float(vb[i]);
        }
      }
      // S buffer can be refilled as soon as every warp has its copy
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[st]);
      const bool need_mask = (kv0 + 64 > de) || (p.causal && kv0 + 63 > q0);
      m_half = -INFINITY;
      if (need_mask) {
        const int lim = p.causal ? min(de - 1, qrow) : de - 1;  // last visible kv index
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const bool vis = row_ok && (kv0 + i <= lim);
          s[i] = vis ? s[i] : -INFINITY;
          m_half = fmaxf(m_half, s[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; i += 2) m_half = fmax3(m_half, s[i], s[i + 1]);
      }
      s_rowmax[((j & 1) * 2 + half) * 128 + row] = m_half;
      return true;
    };
    for (int j = 0; j < nblk; ++j) {
      float s[64];
      float m_half = -INFINITY;
      // a wait that gave up is published before the group barrier, so that all eight warps leave the loop together
      if (!ok || !block(j, s, m_half)) { *s_dead = 1; ok = false; }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (*s_dead) { ok = false; break; }
      const float m_blk = fmaxf(m_half, s_rowmax[((j & 1) * 2 + (half ^ 1)) * 128 + row]);
      mx_logit = fmaxf(mx_logit, m_blk);
      // raise the running maximum only when the block exceeds it by more than AT_LAZY powers of two
      float alpha = 1.f;
      if (m_blk > m_run && (m_run == -INFINITY || (m_blk - m_run) * c > AT_LAZY)) {
        alpha = (m_run == -INFINITY) ? 0.f : fast_exp2((m_run - m_blk) * c);
        m_run = m_blk;
      }
      const float mc = (m_run == -INFINITY) ? 0.f : m_run * c;
      // O may only be touched once the previous P.V has retired (rare: only when a row maximum was raised)
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        if (!mbar_wait(&p_empty[(j - 1) & 1], ((j - 1) >> 1) & 1, KID_ATTN_FWD, 10)) { ok = false; continue; }
        tc_fence_after();
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {
          uint32_t v[32];
          const uint32_t t_o = tm_O + half * 64 + cb * 32 + lane_off;
          tmem_ld_32x32b_x32(t_o, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32b_x32(t_o, v);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      // this P buffer was read by the P.V of two blocks ago
      if (j > 1) {
        if (!mbar_wait(&p_empty[j & 1], ((j >> 1) & 1) ^ 1, KID_ATTN_FWD, 12)) { ok = false; continue; }
        tc_fence_after();
      }
      // two columns per instruction: exponent argument, row-sum accumulation (of the unrounded probabilities)
      const uint64_t cc = f2_pack(c, c), nmc = f2_pack(-mc, -mc);
      uint64_t l2 = f2_pack(0.f, 0.f);
      uint32_t w[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float a0, a1;
        f2_unpack(f2_fma(f2_pack(s[2 * i], s[2 * i + 1]), cc, nmc), a0, a1);
        const float e0 = fast_exp2(a0), e1 = fast_exp2(a1);
        w[i] = pack_bf16(e0, e1);
        l2 = f2_add(l2, f2_pack(e0, e1));
      }
      tmem_st_32x32b_x32(tm_P + (j & 1) * 64 + half * 32 + lane_off, w);
      tmem_st_wait();
      float l_lo, l_hi;
      f2_unpack(l2, l_lo, l_hi);
      const float l_blk = l_lo + l_hi;
      l_run = l_run * alpha + l_blk;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: both halves' row sums, then each half normalises and stores its 64 output columns
    s_rowsum[half * 128 + row] = l_run;
    if (ok && nblk > 0) ok = mbar_wait(&p_empty[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, KID_ATTN_FWD, 11);
    if (!ok) *s_dead = 1;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (*s_dead) ok = false;
    const float l = s_rowsum[row] + s_rowsum[128 + row];
    if (ok && row_ok && half == 0) {
      if (p.lse) p.lse[static_cast<long long>(h) * p.T + qrow] = (l > 0.f) ? m_run * p.scale + logf(l) : -INFINITY;
    }
    if (p.max_logit && half == 0) {
      float wm = warp_max(row_ok ? mx_logit * p.scale : -INFINITY);
      if (lane == 0 && wm > -INFINITY) atomic_max_float(&p.max_logit[h], wm);
    }
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (static_cast<long long>(qrow) * p.Hq + h) * AT_D + half * 64;
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
        uint32_t v[32];
        if (nblk > 0) {
          tmem_ld_32x32b_x32(tm_O + half * 64 + cb * 32 + lane_off, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + cb * 32 + i) = w;
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

template <int DQK>
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnFwdParams& p, int n_tiles,
                           cudaStream_t stream) {
  static bool smem_done[16] = {};
  const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(attn_fwd_kernel<DQK>), AttnSmem<DQK>::TOTAL, smem_done);
  if (e != cudaSuccess) return 300 + static_cast<int>(e);
  dim3 grid(p.Hq, n_tiles);
  attn_fwd_kernel<DQK><<<grid, 320, AttnSmem<DQK>::TOTAL, stream>>>(tq, tk, tv, p);
  return 0;
}

static int make_rows_map(CUtensorMap* m, const void* base, long long rows, long long row_stride_elems, int cols) {
  uint64_t dims[2] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows)};
  uint64_t str[1] = {static_cast<uint64_t>(row_stride_elems) * 2};
  uint32_t box[2] = {64, 128};
  return make_tmap_bf16(m, base, 2, dims, str, box);
}

}  // namespace ttb

using namespace ttb;

// q: [T, Hq*D] (row stride ldq), k: [T, Hk*D] (ldk), v: [T, Hk*128] (ldv; may be a strided view); D = 128 or 192
TTB_EXPORT int ttb_attn_fwd(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                            void* out, float* lse, float* max_logit, const int* q_tiles, int n_tiles, long long T,
                            int Hq, int Hk, int D, float scale, int causal, void* stream) {
  if ((D != 128 && D != 192) || Hq % Hk) return 901;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8)) return 902;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) return 903;
  if (n_tiles == 0) return 0;
  CUtensorMap tq, tk, tv;
  if (make_rows_map(&tq, q, T, ldq, Hq * D)) return 101;
  if (make_rows_map(&tk, k, T, ldk, Hk * D)) return 102;
  if (make_rows_map(&tv, v, T, ldv, Hk * AT_D)) return 103;
  AttnFwdParams p{q_tiles, (__nv_bfloat16*)out, lse, max_logit, Hq, Hk, T, scale, causal};
  const int rc = D == 128 ? launch_attn_fwd<128>(tq, tk, tv, p, n_tiles, reinterpret_cast<cudaStream_t>(stream))
                          : launch_attn_fwd<192>(tq, tk, tv, p, n_tiles, reinterpret_cast<cudaStream_t>(stream));
  if (rc) return rc;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

TTB_EXPORT int ttb_attn_status(unsigned int* out4, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out4, ttb::g_status_word, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) return (int)e;
  if (reset) {
    unsigned int z[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(ttb::g_status_word, z, sizeof(z));
  }
  return (int)e;
}
