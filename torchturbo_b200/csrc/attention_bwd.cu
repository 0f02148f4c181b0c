// Variable-length flash attention backward for sm_100a (GQA, causal or full; value heads 128 wide, query / key heads
// 128 wide, or 192 for multi-head latent attention).  The kernel is built in two forms: with the dQ^T product and its
// reduction (128-wide heads, the default), and without it, where dQ comes from the query-major pass in
// attention_bwd_dq.cu (192-wide heads, whose accumulators do not fit tensor memory together, and the bit-reproducible
// mode of 128-wide heads).
//
// One CTA owns one 128-row KV tile of one document for one *query* head; K_j and V_j stay resident in shared memory
// and dK_j / dV_j accumulate in TMEM over every 64-row query tile that can see the KV tile.  With grouped-query
// attention the CTAs of the query heads that share a KV head add their dK / dV into fp32 accumulators with vector
// atomics (splitting by query head keeps the longest CTA short: a causal KV tile near the start of a long document
// is seen by every later query tile).  Per query-tile iteration, all on tcgen05 with M = 128:
//     S^T  = K_j  Q_i^T          [kv, q]     (K-major  x K-major)
//     dP^T = V_j  dO_i^T         [kv, q]     (K-major  x K-major)
//     P^T  = exp2(S^T c - lse_q),  dS^T = P^T (dP^T - Delta_q) scale        (one thread per kv row, bf16 -> smem)
//     dV  += P^T  dO_i           [kv, d]     (K-major  x MN-major)
//     dK  += dS^T Q_i            [kv, d]     (K-major  x MN-major)
//     dQ^T = K_j^T dS^T          [d, q]      (MN-major x MN-major)  -> transposed through shared memory and added
//                                            into the fp32 dQ buffer by one TMA reduction per tile (the L2 does the adds)
// Warp roles: 0 TMA producer, 1 MMA issuer, 2-9 softmax/dS, 10-13 dQ read-out.  The softmax of a tile is the longest
// dependent chain of an iteration (TMEM read, 64 exponentials per kv row, two bf16 tiles to shared memory), so two
// warpgroups share it: warps 2-5 take query columns 0-31 of every kv row, warps 6-9 columns 32-63 (a warp may read
// the TMEM lanes 32 (warp % 4) .. +31 at any column).  P^T / dS^T (shared memory) and dQ^T (TMEM) are double-buffered:
// the softmax warps of query tile i+1 run while the tensor cores still consume the P^T / dS^T of tile i, and the dQ
// read-out of tile i overlaps the dQ^T MMAs of tile i+1.  Waits are bounded; on timeout the roles drain to the final
// barrier, TMEM is freed and the status word records where the wait gave up.
//
// Replaces flash-attn 2's backward used through the reference attention interface
// (models/modules/attention/interface.py:114-158).
#include "common.cuh"

namespace ttb {

constexpr unsigned KID_ATTN_BWD = 4;
constexpr int BW_KV = 128;   // kv rows per CTA
constexpr int BW_Q = 64;     // query rows per iteration
constexpr int BW_D = 128;

struct AttnBwdParams {
  const int* kv_tiles;   // [n_tiles, 3]: first kv row, document start, document end
  const float* lse;      // [Hq, T]
  const float* delta;    // [Hq, T]  rowsum(dO * O)
  float* dq_acc;         // [T, Hq, D] fp32, zero-initialised
  __nv_bfloat16* dk;     // [T, Hk, D]   written directly when Hq == Hk
  __nv_bfloat16* dv;     // [T, Hk, D]
  float* dk_acc;         // [T, Hk, D] fp32, zero-initialised (used when Hq > Hk)
  float* dv_acc;
  int Hq, Hk;
  long long T;
  float scale;
  int causal;
  int group_loop;   // 1: one CTA per kv head loops over the query heads of its group (no atomics on dK / dV)
};

template <int DQK, bool WITH_DQ>
struct BwdSmem {
  static constexpr int K_BYTES = 128 * DQK * 2;     // K tile: DQK / 64 panels of 16 KB
  static constexpr int Q_BYTES = 64 * DQK * 2;      // Q tile: DQK / 64 panels of 8 KB
  static constexpr int K = 0;
  static constexpr int V = K + K_BYTES;             // 32 KB
  static constexpr int Q0 = V + 32768;              // 2 x Q_BYTES
  static constexpr int DO0 = Q0 + 2 * Q_BYTES;      // 2 x 16 KB
  static constexpr int PT = DO0 + 2 * 16384;        // 2 x 16 KB  P^T  [128 kv][64 q]
  static constexpr int DST = PT + 2 * 16384;        // 2 x 16 KB  dS^T [128 kv][64 q]
  static constexpr int DQS = DST + 2 * 16384;       // 32 KB  dQ tile [64 q][128 d] fp32, source of the TMA reduction
  static constexpr int LSE = DQS + (WITH_DQ ? 32768 : 0);   // float [2][64]
  static constexpr int DELTA = LSE + 2 * 64 * 4;    // float [2][64]
  static constexpr int BARS = DELTA + 2 * 64 * 4;
  static constexpr int TOTAL = BARS + 256 + 1024;
};

__device__ __forceinline__ float bw_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Warp-collective: 32 consecutive fp32 columns of two accumulators, both loads in flight before the one wait.
__device__ __forceinline__ void tmem_ld32x2(uint32_t ta, uint32_t tb, float (&a)[32], float (&b)[32]) {
  uint32_t va[32], vb[32];
  tmem_ld_32x32b_x32(ta, va);
  tmem_ld_32x32b_x32(tb, vb);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    a[i] = __uint_as_float(va[i]);
    b[i] = __uint_as_float(vb[i]);
  }
}

// Warp-collective: 64 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&out)[64]) {
#pragma unroll
  for (int cb = 0; cb < 2; ++cb) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + cb * 32, v);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) out[cb * 32 + i] = __uint_as_float(v[i]);
  }
}

template <int DQK, bool WITH_DQ>
__global__ void __launch_bounds__(448, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                const __grid_constant__ CUtensorMap tmDQ, const AttnBwdParams p) {
  static_assert(DQK == 128 || !WITH_DQ, "the fused dQ path exists for 128-wide heads only");
  using BwdSmem = ttb::BwdSmem<DQK, WITH_DQ>;
  constexpr int NP = DQK / 64, Q_BYTES = BwdSmem::Q_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BwdSmem::BARS);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;    // [2]
  uint64_t* qdo_empty = bars + 3;   // [2]
  uint64_t* st_full = bars + 5;
  uint64_t* st_empty = bars + 6;
  uint64_t* pds_full = bars + 7;    // [2]
  uint64_t* pds_empty = bars + 9;   // [2]
  uint64_t* dq_full = bars + 11;    // [2]
  uint64_t* dq_empty = bars + 13;   // [2]
  uint64_t* acc_full = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* s_dead = reinterpret_cast<volatile int*>(bars + 17);   // a softmax warp's wait gave up
  volatile int* s_dead_dq = reinterpret_cast<volatile int*>(bars + 18);  // a dQ warp's wait gave up
  float* s_lse = reinterpret_cast<float*>(smem + BwdSmem::LSE);
  float* s_delta = reinterpret_cast<float*>(smem + BwdSmem::DELTA);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Launch order.  With dQ in this kernel, tiles vary fastest: the CTAs of one head run together and share its Q / dO
  // rows in the L2 (with heads fastest the 64K-token backward was 12 % slower).  Without dQ (the query-major pass
  // follows), heads vary fastest as in the forward kernel, so the longest tiles of every head start first: measured
  // 10 % faster at 8192 tokens, equal at 65536.
  const int tile = WITH_DQ ? blockIdx.x : blockIdx.y;
  const int head = WITH_DQ ? blockIdx.y : blockIdx.x;
  const int G = p.Hq / p.Hk;
  // default: one CTA per query head (parallel, dK / dV of a group summed with atomics); group loop: one CTA per kv head
  // walks the query heads of its group one after the other and owns dK / dV alone
  const int hk = p.group_loop ? head : head / G;
  const int hq = p.group_loop ? hk * G : head;
  const int kv0 = p.kv_tiles[tile * 3 + 0];
  const int ds = p.kv_tiles[tile * 3 + 1];
  const int de = p.kv_tiles[tile * 3 + 2];
  // query tiles (64 rows, aligned to the document start) that can see this kv tile
  const int q_first = p.causal ? ds + ((kv0 - ds) / BW_Q) * BW_Q : ds;
  const int n_qt = (de - q_first + BW_Q - 1) / BW_Q;
  const int n_it = p.group_loop ? n_qt * G : n_qt;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
    mbar_init(st_full, 1); mbar_init(st_empty, 8);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&pds_full[i], 8); mbar_init(&pds_empty[i], 1);
      mbar_init(&dq_full[i], 1); mbar_init(&dq_empty[i], 4);
    }
    mbar_init(acc_full, 1);
    *s_dead = 0;
    *s_dead_dq = 0;
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
  const uint32_t tm_ST = tmem_base;          // 64 cols
  const uint32_t tm_DPT = tmem_base + 64;    // 64 cols
  const uint32_t tm_DQT = tmem_base + 128;   // 2 x 64 cols (form with dQ)
  const uint32_t tm_DV = tmem_base + (WITH_DQ ? 256 : 128);    // 128 cols
  const uint32_t tm_DK = tmem_base + (WITH_DQ ? 384 : 256);    // DQK cols

  auto it_head = [&](int it) { return p.group_loop ? hq + it / n_qt : hq; };
  auto it_q0 = [&](int it) { return q_first + (p.group_loop ? it % n_qt : it) * BW_Q; };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmDO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(kv_full, BwdSmem::K_BYTES + 32768);
#pragma unroll
      for (int pn = 0; pn < NP; ++pn) tma_load_2d(smem + BwdSmem::K + pn * 16384, &tmK, kv_full, hk * DQK + pn * 64, kv0);
      tma_load_2d(smem + BwdSmem::V, &tmV, kv_full, hk * BW_D, kv0);
      tma_load_2d(smem + BwdSmem::V + 16384, &tmV, kv_full, hk * BW_D + 64, kv0);
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&qdo_empty[st], ph ^ 1, KID_ATTN_BWD, 1)) break;
        const int h = it_head(it), q0 = it_q0(it);
        mbar_expect_tx(&qdo_full[st], Q_BYTES + 16384);
        uint8_t* sq = smem + BwdSmem::Q0 + st * Q_BYTES;
        uint8_t* sd = smem + BwdSmem::DO0 + st * 16384;
#pragma unroll
        for (int pn = 0; pn < NP; ++pn) tma_load_2d(sq + pn * 8192, &tmQ, &qdo_full[st], h * DQK + pn * 64, q0);
        tma_load_2d(sd, &tmDO, &qdo_full[st], h * BW_D, q0);
        tma_load_2d(sd + 8192, &tmDO, &qdo_full[st], h * BW_D + 64, q0);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t id_s = make_idesc_bf16(128, 64, false, false);
      constexpr uint32_t id_acc = make_idesc_bf16(128, 128, false, true);
      constexpr uint32_t id_dk = make_idesc_bf16(128, DQK, false, true);
      constexpr uint32_t id_dq = make_idesc_bf16(128, 64, true, true);
      const uint32_t sK = smem_u32(smem + BwdSmem::K), sV = smem_u32(smem + BwdSmem::V);
      const uint32_t sPT = smem_u32(smem + BwdSmem::PT), sDST = smem_u32(smem + BwdSmem::DST);
      bool ok = mbar_wait(kv_full, 0, KID_ATTN_BWD, 2);
      auto issue_scores = [&](int it) -> bool {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&qdo_full[st], ph, KID_ATTN_BWD, 3)) return false;
        if (!mbar_wait(st_empty, (it & 1) ^ 1, KID_ATTN_BWD, 4)) return false;
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + BwdSmem::Q0 + st * Q_BYTES);
        const uint32_t sDO = smem_u32(smem + BwdSmem::DO0 + st * 16384);
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk) {  // reduction over the query / key head width
          const uint32_t offa = (kk >> 2) * 16384 + (kk & 3) * 32;   // K / V tiles: [128 rows][64 d] panels
          const uint32_t offb = (kk >> 2) * 8192 + (kk & 3) * 32;    // Q / dO tiles: [64 rows][64 d] panels
          umma_ss(tm_ST, make_smem_desc(sK + offa, 16, 1024), make_smem_desc(sQ + offb, 16, 1024), id_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t offa = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t offb = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_ss(tm_DPT, make_smem_desc(sV + offa, 16, 1024), make_smem_desc(sDO + offb, 16, 1024), id_s, kk != 0);
        }
        umma_commit(st_full);
        return true;
      };
      if (ok && n_it > 0) ok = issue_scores(0);
      for (int it = 0; it < n_it && ok; ++it) {
        if (it + 1 < n_it) {
          if (!issue_scores(it + 1)) { ok = false; break; }
        }
        const int st = it & 1;
        const uint32_t ph2 = (it >> 1) & 1;
        if (!mbar_wait(&pds_full[st], ph2, KID_ATTN_BWD, 5)) { ok = false; break; }
        if (WITH_DQ) {
          if (!mbar_wait(&dq_empty[st], ph2 ^ 1, KID_ATTN_BWD, 6)) { ok = false; break; }
        }
        tc_fence_after();
        const uint32_t sPTb = sPT + st * 16384, sDSTb = sDST + st * 16384;
        const uint32_t sQ = smem_u32(smem + BwdSmem::Q0 + st * Q_BYTES);
        const uint32_t sDO = smem_u32(smem + BwdSmem::DO0 + st * 16384);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {  // reduction over q = 64
          // A: P^T / dS^T K-major single panel; B: dO / Q as [q rows][d] MN-major, d panels 8 KB apart
          umma_ss(tm_DV, make_smem_desc(sPTb + kk * 32, 16, 1024), make_smem_desc(sDO + kk * 2048, 8192, 1024), id_acc,
                  (it | kk) != 0);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          umma_ss(tm_DK, make_smem_desc(sDSTb + kk * 32, 16, 1024), make_smem_desc(sQ + kk * 2048, 8192, 1024), id_dk,
                  (it | kk) != 0);
        }
        umma_commit(&qdo_empty[st]);
        if (WITH_DQ) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {  // reduction over kv = 128
            // A: K^T from the K tile ([kv rows][d], MN-major, d panels 16 KB apart); B: dS^T ([kv rows][q]) MN-major
            umma_ss(tm_DQT + st * 64, make_smem_desc(sK + kk * 2048, 16384, 1024),
                    make_smem_desc(sDSTb + kk * 2048, 8192, 1024), id_dq, kk != 0);
          }
          umma_commit(&dq_full[st]);
        }
        umma_commit(&pds_empty[st]);
      }
      if (ok) umma_commit(acc_full);
    }
  } else if (warp < 10) {
    // ---------------------------------------------------------------- softmax / dS (thread = kv row, 32 query columns)
    const int lg = warp & 3;
    const int half = (warp - 2) >> 2;          // 0: query columns 0-31, 1: columns 32-63
    const int row = lg * 32 + lane;
    const int kv = kv0 + row;
    const bool kv_ok = kv < de;
    const float c = p.scale * 1.4426950408889634f;
    const int tid = threadIdx.x - 64;  // 0..255 inside the two groups
    bool ok = true;
    // lse / delta of the 64 query rows of an iteration are staged one iteration ahead (double-buffered); the global
    // load is issued at the top of the iteration before and stored at its end
    auto fetch = [&](int it) -> float {
      const int q0s = it_q0(it);
      if (tid < 64) {
        const int q = q0s + tid;
        return (q < de) ? -p.lse[static_cast<long long>(it_head(it)) * p.T + q] * 1.4426950408889634f : -INFINITY;
      }
      if (tid < 128) {
        const int q = q0s + tid - 64;
        return (q < de) ? -p.delta[static_cast<long long>(it_head(it)) * p.T + q] * p.scale : 0.f;
      }
      return 0.f;
    };
    auto put = [&](int it, float v) {
      if (tid < 64) s_lse[(it & 1) * 64 + tid] = v;
      else if (tid < 128) s_delta[(it & 1) * 64 + tid - 64] = v;
    };
    if (n_it > 0) put(0, fetch(0));
    asm volatile("bar.sync 1, 256;" ::: "memory");
    // one iteration; false when a wait gave up (the caller still joins the group barrier, so no warp is left in it)
    auto body = [&](int it) -> bool {
      const int q0 = it_q0(it);
      const float staged = (it + 1 < n_it) ? fetch(it + 1) : 0.f;
      if (!mbar_wait(st_full, it & 1, KID_ATTN_BWD, 7)) return false;
      tc_fence_after();
      float s[32], dp[32];
      const uint32_t lane_off = (static_cast<uint32_t>(lg * 32) << 16) + half * 32;
      tmem_ld32x2(tm_ST + lane_off, tm_DPT + lane_off, s, dp);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(st_empty);
      const float* lse = s_lse + (it & 1) * 64 + half * 32;
      const float* dl = s_delta + (it & 1) * 64 + half * 32;
      const int qh = q0 + half * 32;
      const bool need_mask = (q0 + BW_Q > de) || (kv0 + BW_KV > de) || (p.causal && kv0 + BW_KV - 1 > qh);
      // the tile that used this P^T / dS^T buffer two iterations ago must have been consumed (a fresh barrier passes)
      if (!mbar_wait(&pds_empty[it & 1], ((it >> 1) & 1) ^ 1, KID_ATTN_BWD, 8)) return false;
      uint8_t* sPT = smem + BwdSmem::PT + (it & 1) * 16384;
      uint8_t* sDST = smem + BwdSmem::DST + (it & 1) * 16384;
      // two columns per instruction; the staged row statistics are -lse log2(e) and -Delta scale
      const uint64_t cc = f2_pack(c, c), sc2 = f2_pack(p.scale, p.scale);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t wp[4], wd[4];
        const ulonglong2 l01 = *reinterpret_cast<const ulonglong2*>(lse + ch * 8), l23 = *reinterpret_cast<const ulonglong2*>(lse + ch * 8 + 4);
        const ulonglong2 d01 = *reinterpret_cast<const ulonglong2*>(dl + ch * 8), d23 = *reinterpret_cast<const ulonglong2*>(dl + ch * 8 + 4);
        const uint64_t lv[4] = {l01.x, l01.y, l23.x, l23.y};
        const uint64_t dlv[4] = {d01.x, d01.y, d23.x, d23.y};
#pragma unroll
        for (int qq = 0; qq < 4; ++qq) {
          const int col = ch * 8 + qq * 2;
          float a0, a1;
          f2_unpack(f2_fma(f2_pack(s[col], s[col + 1]), cc, lv[qq]), a0, a1);
          float p0 = bw_exp2(a0), p1 = bw_exp2(a1);
          if (need_mask) {
            const int q = qh + col;
            p0 = (kv_ok && q < de && (!p.causal || kv <= q)) ? p0 : 0.f;
            p1 = (kv_ok && q + 1 < de && (!p.causal || kv <= q + 1)) ? p1 : 0.f;
          }
          float d0, d1;
          f2_unpack(f2_mul(f2_pack(p0, p1), f2_fma(f2_pack(dp[col], dp[col + 1]), sc2, dlv[qq])), d0, d1);
          wp[qq] = pack_bf16(p0, p1);
          wd[qq] = pack_bf16(d0, d1);
        }
        const int off = row * 128 + (((half * 4 + ch) ^ (row & 7)) * 16);
        *reinterpret_cast<uint4*>(sPT + off) = make_uint4(wp[0], wp[1], wp[2], wp[3]);
        *reinterpret_cast<uint4*>(sDST + off) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[it & 1]);
      if (it + 1 < n_it) put(it + 1, staged);
      return true;
    };
    for (int it = 0; it < n_it; ++it) {
      if (!body(it)) { *s_dead = 1; ok = false; }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (*s_dead) { ok = false; break; }
    }
    // ---- epilogue: dK / dV of this tile
    if (ok && n_it > 0) ok = mbar_wait(acc_full, 0, KID_ATTN_BWD, 9);
    if (ok) {
      tc_fence_after();
      const uint32_t lane_off = static_cast<uint32_t>(lg * 32) << 16;
      {
        const int which = half;                  // columns 0-31 group: dV, the other group: dK
        const int width = which == 0 ? BW_D : DQK;
        const long long off = (static_cast<long long>(kv) * p.Hk + hk) * width;
        __nv_bfloat16* dst = (which == 0 ? p.dv : p.dk) + off;
        float* acc = (which == 0 ? p.dv_acc : p.dk_acc) + off;
        const uint32_t tm = (which == 0 ? tm_DV : tm_DK) + lane_off;
#pragma unroll 1
        for (int cb = 0; cb < width / 32; ++cb) {
          uint32_t v[32];
          if (n_it > 0) {
            tmem_ld_32x32b_x32(tm + cb * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          if (kv_ok) {
            if (G == 1 || p.group_loop) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 w;
                w.x = pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                w.y = pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                w.z = pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                w.w = pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                *reinterpret_cast<uint4*>(dst + cb * 32 + i) = w;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                atomicAdd(reinterpret_cast<float4*>(acc + cb * 32 + i),
                          make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]),
                                      __uint_as_float(v[i + 3])));
              }
            }
          }
        }
      }
    }
  } else if (WITH_DQ) {
    // ---------------------------------------------------------------- dQ read-out (thread = head-dim index d)
    const int lg = warp & 3;                    // warps 10-13: TMEM lane groups 2, 3, 0, 1
    const int d = lg * 32 + lane;
    const int tid_dq = threadIdx.x - 320;       // 0..127
    float* sdq = reinterpret_cast<float*>(smem + BwdSmem::DQS);
    bool alive = true;
    if (tid_dq == 0) tma_prefetch_desc(&tmDQ);
    for (int it = 0; it < n_it; ++it) {
      const int q0 = it_q0(it);
      float v[64];
      if (alive && !mbar_wait(&dq_full[it & 1], (it >> 1) & 1, KID_ATTN_BWD, 10)) { alive = false; *s_dead_dq = 1; }
      if (alive) {
        tc_fence_after();
        tmem_ld64(tm_DQT + (it & 1) * 64 + (static_cast<uint32_t>(lg * 32) << 16), v);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&dq_empty[it & 1]);
      }
      // the reduction of the previous tile has finished reading the staging tile
      if (it > 0 && tid_dq == 0) bulk_wait_read_all();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (*s_dead_dq) break;
      // transpose: this thread's d column of the [64 q][128 d] tile (a warp writes 128 contiguous bytes per row).
      // Query rows past the end of the document carry exact zeros (their P and dS were masked), so the full tile
      // is added; rows past the end of the tensor are clipped by the copy engine.
#pragma unroll
      for (int col = 0; col < BW_Q; ++col) sdq[col * BW_D + d] = v[col];
      fence_proxy_async_smem();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (tid_dq == 0) {
        tma_reduce_add_2d(&tmDQ, sdq, hq * BW_D, q0);
        bulk_commit_group();
      }
    }
    if (tid_dq == 0) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]; also converts nothing else.  One warp per (t, h).
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                      float* __restrict__ delta, long long T, int Hq) {
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= T * Hq) return;
  const long long t = gw / Hq;
  const int h = static_cast<int>(gw - t * Hq);
  const uint2 a = *reinterpret_cast<const uint2*>(dout + gw * BW_D + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(out + gw * BW_D + lane * 4);
  const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y);
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  s = warp_sum(s);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = s;
}

// dq (bf16) = dq_acc (fp32)
__global__ void attn_bwd_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long n) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  const float4 a = *reinterpret_cast<const float4*>(acc + i), b = *reinterpret_cast<const float4*>(acc + i + 4);
  uint4 w;
  w.x = pack_bf16(a.x, a.y); w.y = pack_bf16(a.z, a.w); w.z = pack_bf16(b.x, b.y); w.w = pack_bf16(b.z, b.w);
  *reinterpret_cast<uint4*>(dq + i) = w;
}

static int bw_map(CUtensorMap* m, const void* base, long long rows, long long row_stride, int cols, int box_rows) {
  uint64_t dims[2] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows)};
  uint64_t str[1] = {static_cast<uint64_t>(row_stride) * 2};
  uint32_t box[2] = {64, static_cast<uint32_t>(box_rows)};
  return make_tmap_bf16(m, base, 2, dims, str, box);
}

}  // namespace ttb

using namespace ttb;

template <int DQK, bool WITH_DQ>
static int launch_attn_bwd(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tk, const CUtensorMap& tv,
                           const CUtensorMap& tdq, const AttnBwdParams& p, int n_tiles, cudaStream_t stream) {
  static bool smem_done[16] = {};
  using Smem = ttb::BwdSmem<DQK, WITH_DQ>;
  const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(attn_bwd_kernel<DQK, WITH_DQ>), Smem::TOTAL, smem_done);
  if (e != cudaSuccess) return 300 + static_cast<int>(e);
  const int heads = p.group_loop ? p.Hk : p.Hq;
  dim3 grid(WITH_DQ ? n_tiles : heads, WITH_DQ ? heads : n_tiles);
  attn_bwd_kernel<DQK, WITH_DQ><<<grid, WITH_DQ ? 448 : 320, Smem::TOTAL, stream>>>(tq, tdo, tk, tv, tdq, p);
  return 0;
}

// q: [T, Hq*D] contiguous rows; dout, out: [T, Hq*128] contiguous rows; k: [T, Hk*D] (ldk); v: [T, Hk*128] (ldv, may be
// strided); D = 128 or 192.  delta fp32 [Hq*T] scratch (left filled with rowsum(dO * O) for the query-major dQ pass).
// with_dq != 0 (D = 128 only): dQ too, reduced into dq_acc (fp32 [T*Hq*128], zero-initialised) and cast to dq;
// with_dq == 0: dK and dV only (dq_acc and dq unused); with_dq == 2: the same with one CTA per kv head looping over the
// query heads of its group, so that dK / dV are written once and without atomics (no accumulators needed).  dk: [T, Hk, D], dv: [T, Hk, 128]; with Hq > Hk the fp32
// accumulators dk_acc / dv_acc (zero-initialised, same shapes) are required.
TTB_EXPORT int ttb_attn_bwd(const void* q, const void* k, long long ldk, const void* v, long long ldv, const void* out,
                            const void* dout, const float* lse, float* delta, float* dq_acc, float* dk_acc,
                            float* dv_acc, void* dq, void* dk, void* dv, const int* kv_tiles, int n_tiles, long long T, int Hq, int Hk, int D, float scale,
                            int causal, int with_dq, void* stream_ptr) {
  if ((D != 128 && D != 192) || Hq % Hk) return 901;
  const int group_loop = with_dq == 2;
  if (group_loop) with_dq = 0;
  if (with_dq && D != 128) return 904;
  if ((ldk % 8) || (ldv % 8)) return 902;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  if (T == 0 || n_tiles == 0) return 0;
  const long long warps = T * Hq;
  attn_bwd_delta_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)dout,
                                                                        (const __nv_bfloat16*)out, delta, T, Hq);
  CUtensorMap tq, tdo, tk, tv;
  if (bw_map(&tq, q, T, (long long)Hq * D, Hq * D, 64)) return 101;
  if (bw_map(&tdo, dout, T, (long long)Hq * BW_D, Hq * BW_D, 64)) return 102;
  if (bw_map(&tk, k, T, ldk, Hk * D, 128)) return 103;
  if (bw_map(&tv, v, T, ldv, Hk * BW_D, 128)) return 104;
  CUtensorMap tdq = tq;   // placeholder in the form without dQ
  if (with_dq) {
    if (dq_acc == nullptr || dq == nullptr) return 905;
    uint64_t dims[2] = {static_cast<uint64_t>(Hq) * D, static_cast<uint64_t>(T)};
    uint64_t str[1] = {static_cast<uint64_t>(Hq) * D * 4};
    uint32_t box[2] = {static_cast<uint32_t>(D), 64};
    if (make_tmap_f32_linear(&tdq, dq_acc, 2, dims, str, box)) return 105;
  }
  if (Hq != Hk && !group_loop && (dk_acc == nullptr || dv_acc == nullptr)) return 903;
  AttnBwdParams p{kv_tiles, lse, delta, dq_acc, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, dk_acc, dv_acc, Hq, Hk, T, scale, causal, group_loop};
  const int rc = with_dq ? launch_attn_bwd<128, true>(tq, tdo, tk, tv, tdq, p, n_tiles, stream)
                         : (D == 128 ? launch_attn_bwd<128, false>(tq, tdo, tk, tv, tdq, p, n_tiles, stream)
                                     : launch_attn_bwd<192, false>(tq, tdo, tk, tv, tdq, p, n_tiles, stream));
  if (rc) return rc;
  if (with_dq) {
    const long long n = T * Hq * D;
    attn_bwd_cast_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, stream>>>(dq_acc, (__nv_bfloat16*)dq, n);
  }
  if (Hq != Hk && !group_loop) {
    const long long nk = T * Hk * D, nv = T * Hk * BW_D;
    attn_bwd_cast_kernel<<<(unsigned)((nk / 8 + 255) / 256), 256, 0, stream>>>(dk_acc, (__nv_bfloat16*)dk, nk);
    attn_bwd_cast_kernel<<<(unsigned)((nv / 8 + 255) / 256), 256, 0, stream>>>(dv_acc, (__nv_bfloat16*)dv, nv);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
