// Chunk-state recurrence of the (gated) delta rule for sm_100a: the only sequential part of the chunked evaluation of
// GatedDeltaNet / Kimi Delta Attention layers, forward and backward.
//
// With 64-token chunks and per-chunk operands prepared by chunk-parallel (batched) GEMMs, the state S [K=128, V=128] of
// one head of one sequence obeys
//     X_c     = U_c  + s1 * A_c S            [64, V]     forward:  v_new = u - w S            (s1 = -1, A = w)
//     S      <- d_c (.) S + s2 * B_c^T X_c   [K, V]      forward:  S = d S + k_out^T v_new    (s2 = +1, B = k_out)
// and the reverse pass over the same chunks has the same shape with the operands swapped,
//     dX_c    = G_c  + k_out_c dS            (s1 = +1, A = k_out, U = gradient that reaches v_new directly)
//     dS     <- d_c (.) dS - w_c^T dX_c + GS_c   (s2 = -1, B = w, GS = gradient that reaches the chunk's start state)
// so one kernel runs both directions.  d_c is a scalar per chunk (GatedDeltaNet) or a vector over K (KDA).
//
// One CTA owns one (sequence, head).  The state lives transposed in registers, one thread per value column v holding
// its 128 K-entries in fp32 (TMEM lane = v), and as a bf16 K-major tile in shared memory for the tensor cores:
//     acc1 [V, 64]  = S^T  A_c^T       tcgen05, M = 128, N = 64   (K-major x K-major)
//     acc2 [V, 128] = X^T  B_c         tcgen05, M = 128, N = 128  (K-major x MN-major)
// Warp roles: 0 TMA producer (A_c / B_c tiles, two stages), 1 MMA issuer, 2-5 state warps.  Every wait is bounded; on a
// timeout the roles drain to the final barrier, TMEM is freed and the status word records kernel / site.
//
// Counterpart of the `chunk_gated_delta_rule` / `chunk_kda` operators that the reference takes from
// flash-linear-attention (ops/providers/native/gated_delta_rule.py, ops/providers/native/kda.py).
#include "common.cuh"

namespace ttb {

constexpr unsigned KID_DELTA_STATE = 9;
constexpr int DS_C = 64;     // tokens per chunk
constexpr int DS_D = 128;    // K = V = 128

struct DeltaStateParams {
  const float* U;        // [H, NC, 64, 128]
  float* X;              // [H, NC, 64, 128]
  const float* decay;    // [H, NC] or [H, NC, 128]
  const float* init;     // [H, nseq, 128, 128] or null (zeros)
  const float* add;      // [H, NC + nseq, 128, 128] or null
  float* states;         // [H, NC + nseq, 128, 128]
  const int* seq_chunks; // [nseq, 2]: first chunk, number of chunks
  int nseq, H, NC;
  int vec, reverse;
  float s1, s2;
};

struct DsSmem {
  static constexpr int ST = 0;                      // S^T bf16 [128 v][128 k]: 2 panels of 16 KB
  static constexpr int XT = ST + 32768;             // X^T bf16 [128 v][64 c]: 16 KB
  static constexpr int A0 = XT + 16384;             // 2 x 16 KB  A_c [64 c][128 k]
  static constexpr int B0 = A0 + 2 * 16384;         // 2 x 16 KB  B_c [64 c][128 k]
  static constexpr int DEC = B0 + 2 * 16384;        // float [128]
  static constexpr int BARS = DEC + 512;
  static constexpr int TOTAL = BARS + 256 + 1024;
};

__global__ void __launch_bounds__(192, 1)
delta_state_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const DeltaStateParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DsSmem::BARS);
  uint64_t* ab_full = bars + 0;     // [2]
  uint64_t* ab_empty = bars + 2;    // [2]
  uint64_t* st_ready = bars + 4;    // S^T (bf16) of the next chunk is in shared memory
  uint64_t* acc1_full = bars + 5;
  uint64_t* x_ready = bars + 6;     // X^T (bf16) is in shared memory
  uint64_t* acc2_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* s_dead = reinterpret_cast<volatile int*>(bars + 9);
  float* s_dec = reinterpret_cast<float*>(smem + DsSmem::DEC);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.x, h = blockIdx.y;
  const int c0 = p.seq_chunks[seq * 2 + 0];
  const int n = p.seq_chunks[seq * 2 + 1];
  const int slots = p.NC + p.nseq;
  auto chunk_of = [&](int i) { return p.reverse ? c0 + n - 1 - i : c0 + i; };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&ab_full[i], 1); mbar_init(&ab_empty[i], 1); }
    mbar_init(st_ready, 4);
    mbar_init(acc1_full, 1);
    mbar_init(x_ready, 4);
    mbar_init(acc2_full, 1);
    *s_dead = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm1 = tmem_base;         // 64 columns
  const uint32_t tm2 = tmem_base + 128;   // 128 columns

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB);
      for (int i = 0; i < n; ++i) {
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&ab_empty[st], ph ^ 1, KID_DELTA_STATE, 1)) break;
        const int row0 = (h * p.NC + chunk_of(i)) * DS_C;
        mbar_expect_tx(&ab_full[st], 32768);
        uint8_t* sa = smem + DsSmem::A0 + st * 16384;
        uint8_t* sb = smem + DsSmem::B0 + st * 16384;
        tma_load_2d(sa, &tmA, &ab_full[st], 0, row0);
        tma_load_2d(sa + 8192, &tmA, &ab_full[st], 64, row0);
        tma_load_2d(sb, &tmB, &ab_full[st], 0, row0);
        tma_load_2d(sb + 8192, &tmB, &ab_full[st], 64, row0);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t id1 = make_idesc_bf16(128, 64, false, false);
      constexpr uint32_t id2 = make_idesc_bf16(128, 128, false, true);
      const uint32_t sST = smem_u32(smem + DsSmem::ST), sXT = smem_u32(smem + DsSmem::XT);
      for (int i = 0; i < n; ++i) {
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&ab_full[st], ph, KID_DELTA_STATE, 2)) break;
        if (!mbar_wait(st_ready, i & 1, KID_DELTA_STATE, 3)) break;
        tc_fence_after();
        const uint32_t sA = smem_u32(smem + DsSmem::A0 + st * 16384);
        const uint32_t sB = smem_u32(smem + DsSmem::B0 + st * 16384);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // reduction over k = 128
          umma_ss(tm1, make_smem_desc(sST + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                  make_smem_desc(sA + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), id1, kk != 0);
        }
        umma_commit(acc1_full);
        if (!mbar_wait(x_ready, i & 1, KID_DELTA_STATE, 4)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {  // reduction over the 64 tokens of the chunk
          umma_ss(tm2, make_smem_desc(sXT + kk * 32, 16, 1024), make_smem_desc(sB + kk * 2048, 8192, 1024), id2, kk != 0);
        }
        umma_commit(acc2_full);
        umma_commit(&ab_empty[st]);
      }
    }
  } else {
    // ---------------------------------------------------------------- state warps (thread = value column v)
    const int lg = warp & 3;
    const int v = lg * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(lg * 32) << 16;
    const int tid = threadIdx.x - 64;
    float S[DS_D];
    uint8_t* sST = smem + DsSmem::ST;
    uint8_t* sXT = smem + DsSmem::XT;
    auto state_ptr = [&](const float* base, int slot) {
      return base + ((static_cast<long long>(h) * slots + slot) * DS_D) * DS_D + v;
    };
    // S^T row v -> bf16 K-major tile (two 64-wide panels, 128-byte swizzle)
    auto publish = [&]() {
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        uint4 w;
        w.x = pack_bf16(S[ch * 8 + 0], S[ch * 8 + 1]); w.y = pack_bf16(S[ch * 8 + 2], S[ch * 8 + 3]);
        w.z = pack_bf16(S[ch * 8 + 4], S[ch * 8 + 5]); w.w = pack_bf16(S[ch * 8 + 6], S[ch * 8 + 7]);
        *reinterpret_cast<uint4*>(sST + (ch >> 3) * 16384 + v * 128 + (((ch & 7) ^ (v & 7)) * 16)) = w;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(st_ready);
    };
    // initial state, also recorded in the slot that precedes the first processed chunk
    {
      const int slot0 = (p.reverse ? c0 + n : c0) + seq;
      const float* src = p.reverse ? (p.add ? state_ptr(p.add, slot0) : nullptr)
                                   : (p.init ? p.init + ((static_cast<long long>(h) * p.nseq + seq) * DS_D) * DS_D + v : nullptr);
      float* dst = const_cast<float*>(state_ptr(p.states, slot0));
      // all loads before the first store: the compiler may not move a load above a store that could alias it
#pragma unroll
      for (int k = 0; k < DS_D; ++k) S[k] = src ? src[k * DS_D] : 0.f;
#pragma unroll
      for (int k = 0; k < DS_D; ++k) dst[k * DS_D] = S[k];
    }
    if (n > 0) publish();
    bool ok = true;
    auto step = [&](int i) -> bool {
      const int c = chunk_of(i);
      const long long xoff = ((static_cast<long long>(h) * p.NC + c) * DS_C) * DS_D + v;
      // the chunk in two halves of 32 tokens: U is fetched ahead of the product it is added to
      float u[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) u[j] = p.U[xoff + j * DS_D];
      if (!mbar_wait(acc1_full, i & 1, KID_DELTA_STATE, 5)) return false;
      tc_fence_after();
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tm1 + cb * 32 + lane_off, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) u[j] = fmaf(p.s1, __uint_as_float(r[j]), u[j]);
#pragma unroll
        for (int j = 0; j < 32; ++j) p.X[xoff + (cb * 32 + j) * DS_D] = u[j];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint4 w;
          w.x = pack_bf16(p.s2 * u[ch * 8 + 0], p.s2 * u[ch * 8 + 1]); w.y = pack_bf16(p.s2 * u[ch * 8 + 2], p.s2 * u[ch * 8 + 3]);
          w.z = pack_bf16(p.s2 * u[ch * 8 + 4], p.s2 * u[ch * 8 + 5]); w.w = pack_bf16(p.s2 * u[ch * 8 + 6], p.s2 * u[ch * 8 + 7]);
          *reinterpret_cast<uint4*>(sXT + v * 128 + (((cb * 4 + ch) ^ (v & 7)) * 16)) = w;
        }
        if (cb == 0) {
#pragma unroll
          for (int j = 0; j < 32; ++j) u[j] = p.U[xoff + (32 + j) * DS_D];
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(x_ready);
      // a vector decay is staged for all threads while the second product runs
      if (p.vec) s_dec[tid] = p.decay[(static_cast<long long>(h) * p.NC + c) * DS_D + tid];
      return true;
    };
    for (int i = 0; i < n; ++i) {
      const int c = chunk_of(i);
      if (!ok || !step(i)) { *s_dead = 1; ok = false; }
      asm volatile("bar.sync 1, 128;" ::: "memory");     // the decay vector is staged; a failed wait is published
      if (*s_dead) { ok = false; break; }
      if (!mbar_wait(acc2_full, i & 1, KID_DELTA_STATE, 6)) { ok = false; continue; }
      tc_fence_after();
      const float dsc = p.vec ? 1.f : p.decay[static_cast<long long>(h) * p.NC + c];
      const int slot = (p.reverse ? c : c + 1) + seq;
      const float* addp = p.add ? state_ptr(p.add, slot) : nullptr;
      float* dst = const_cast<float*>(state_ptr(p.states, slot));
#pragma unroll
      for (int cb = 0; cb < 4; ++cb) {
        // the 32 added values are fetched together, ahead of the stores of this block (a load may not pass a store
        // that could alias it, and one exposed memory round trip per value would dominate the chunk)
        float av[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) av[j] = addp ? addp[(cb * 32 + j) * DS_D] : 0.f;
        uint32_t r[32];
        tmem_ld_32x32b_x32(tm2 + cb * 32 + lane_off, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int k = cb * 32 + j;
          const float d = p.vec ? s_dec[k] : dsc;
          S[k] = fmaf(d, S[k], __uint_as_float(r[j])) + av[j];
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[(cb * 32 + j) * DS_D] = S[cb * 32 + j];
      }
      tc_fence_before();
      if (i + 1 < n) publish();
    }
    if (!ok) *s_dead = 1;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace ttb

using namespace ttb;

// A, B: bf16 [H * NC * 64, 128] (chunk-major rows); U, X: fp32 [H, NC, 64, 128]; decay fp32 [H, NC] or [H, NC, 128];
// init fp32 [H, nseq, 128, 128] or null; add, states fp32 [H, NC + nseq, 128, 128] (add may be null when forward).
TTB_EXPORT int ttb_delta_state_scan(const void* A, const void* B, const float* U, float* X, const float* decay, int vec,
                                    const float* init, const float* add, float* states, const int* seq_chunks, int nseq,
                                    int H, int NC, int reverse, float s1, float s2, void* stream_ptr) {
  if (nseq <= 0 || H <= 0 || NC <= 0) return 0;
  if (reverse && add == nullptr) return 911;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_ptr);
  CUtensorMap ta, tb;
  const long long rows = static_cast<long long>(H) * NC * DS_C;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(DS_D), static_cast<uint64_t>(rows)};
    uint64_t str[1] = {static_cast<uint64_t>(DS_D) * 2};
    uint32_t box[2] = {64, 64};
    if (make_tmap_bf16(&ta, A, 2, dims, str, box)) return 101;
    if (make_tmap_bf16(&tb, B, 2, dims, str, box)) return 102;
  }
  static bool smem_done[16] = {};
  {
    const cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(delta_state_kernel), DsSmem::TOTAL, smem_done);
    if (e != cudaSuccess) return 300 + static_cast<int>(e);
  }
  DeltaStateParams p{U, X, decay, init, add, states, seq_chunks, nseq, H, NC, vec, reverse, s1, s2};
  dim3 grid(nseq, H);
  delta_state_kernel<<<grid, 192, DsSmem::TOTAL, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
