// MoE routing and token permutation kernels for sm_100a.
//
//  * router_fwd / router_bwd: one warp per token does the score function
//    (softmax before or after top-k, or sigmoid), bias-for-selection top-k,
//    probability normalisation, the separate bias-free top-k used by the
//    load-balance loss, per-expert score sums / token counts (padding excluded)
//    and the per-token logsumexp for the z-loss; the backward folds the
//    gradients of the routing weights, of the aux loss and of the z-loss into
//    d(logits).  Semantics: models/modules/moe/router.py:164-380,
//    models/modules/moe/utils.py:127-230, models/modules/moe/moe_utils.py:15-72.
//  * permutation: rows ordered by (expert, token), every expert segment padded
//    to a multiple of 128 rows (pad rows are zero) so that the grouped tcgen05
//    GEMM never straddles experts and the host never learns the split sizes.
//    Contract: ops/moe.py:10-46, ops/providers/native/moe_permutation.py:24-126.
#include "common.cuh"

namespace ttb {

constexpr int MAX_E_PER_LANE = 8;  // E <= 256
constexpr int MAX_K = 16;
constexpr int SEG_ALIGN = 128;

enum ScoreFn : int { SOFTMAX_PRE = 0, SOFTMAX_POST = 1, SIGMOID = 2 };

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax warp_argmax(float v, int i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
  return {v, i};
}

// Select top-k of `sel` (values per lane: expert id = j*32 + lane).  Returns ids through out_idx[k]
// (identical on every lane) in descending order.
__device__ __forceinline__ void warp_topk(const float (&sel)[MAX_E_PER_LANE], int epl, int E, int k, int lane,
                                          int (&out_idx)[MAX_K]) {
  unsigned taken = 0;
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      if (j < epl) {
        int e = j * 32 + lane;
        if (e < E && !((taken >> j) & 1u)) {
          float v = sel[j];
          if (!(v == v)) v = -INFINITY;   // NaN never wins a comparison: rank it last instead of selecting nothing
          if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
        }
      }
    }
    ArgMax am = warp_argmax(bv, bi);
    out_idx[r] = am.i;
    if ((am.i & 31) == lane && am.i < E) taken |= 1u << (am.i >> 5);
  }
}

struct RouterParams {
  const float* logits;      // [T, E] fp32
  const float* expert_bias; // [E] or null (selection only)
  const unsigned char* valid_mask;  // [T] or null (1 = real token) - statistics only
  int* topk_idx;            // [T, k]
  float* topk_prob;         // [T, k]
  float* lse;               // [T] or null
  float* score_partial;     // [grid, E] or null : per-block sum of aux scores (valid tokens)
  int* aux_counts;          // [E] or null : tokens per expert from the bias-free top-k (valid tokens)
  int* counts;              // [E] or null : tokens per expert of the routing top-k (all tokens)
  long long T;
  int E, k, score_fn;
  float scaling;
};

__global__ void router_fwd_kernel(const RouterParams p) {
  extern __shared__ float s_scores[];  // [E] block partial
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  const int epl = (p.E + 31) / 32;
  if (p.score_partial) {
    for (int i = threadIdx.x; i < p.E; i += blockDim.x) s_scores[i] = 0.f;
    __syncthreads();
  }
  for (long long t = static_cast<long long>(blockIdx.x) * wpb + wib; t < p.T;
       t += static_cast<long long>(gridDim.x) * wpb) {
    float lg[MAX_E_PER_LANE], sc[MAX_E_PER_LANE], sel[MAX_E_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      int e = j * 32 + lane;
      lg[j] = (j < epl && e < p.E) ? p.logits[t * p.E + e] : -INFINITY;
      mx = fmaxf(mx, lg[j]);
    }
    mx = warp_max(mx);
    float se = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) se += (lg[j] == -INFINITY) ? 0.f : __expf(lg[j] - mx);
    se = warp_sum(se);
    const float lse = mx + logf(se);
    if (p.lse && lane == 0) p.lse[t] = lse;
    // normalised scores used by the aux loss (and by SOFTMAX_PRE / SIGMOID routing)
    float ssum = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      if (lg[j] == -INFINITY) { sc[j] = 0.f; continue; }
      sc[j] = (p.score_fn == SIGMOID) ? 1.f / (1.f + __expf(-lg[j])) : __expf(lg[j] - lse);
      ssum += sc[j];
    }
    if (p.score_fn == SIGMOID) ssum = warp_sum(ssum);
    // selection values
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      int e = j * 32 + lane;
      float base = (p.score_fn == SOFTMAX_POST) ? lg[j] : sc[j];
      if (lg[j] == -INFINITY) base = -INFINITY;
      else if (p.expert_bias) base += p.expert_bias[e];
      // NaN compares false with everything: the selection below would find no candidate and return an index far
      // outside [0, E).  As -inf a NaN row selects the lowest expert ids; its weights stay NaN and reach the loss.
      sel[j] = (base == base) ? base : -INFINITY;
    }
    int idx[MAX_K];
    warp_topk(sel, epl, p.E, p.k, lane, idx);
    // routing weights
    float w = 0.f;  // lane r (< k) holds weight r
    {
      float raw = -INFINITY;
      for (int r = 0; r < p.k; ++r) {
        int e = idx[r];
        // value lives on lane (e & 31), slot (e >> 5): broadcast it
        float vv = 0.f;
#pragma unroll
        for (int j = 0; j < MAX_E_PER_LANE; ++j)
          if (j == (e >> 5)) vv = (p.score_fn == SOFTMAX_POST) ? lg[j] : sc[j];
        vv = __shfl_sync(0xffffffffu, vv, e & 31);
        if (lane == r) raw = vv;
      }
      if (p.score_fn == SOFTMAX_POST) {
        float m2 = warp_max(raw);
        float ex = (lane < p.k) ? __expf(raw - m2) : 0.f;
        float s2 = warp_sum(ex);
        w = ex / s2;
      } else if (p.score_fn == SIGMOID) {
        float v2 = (lane < p.k) ? raw : 0.f;
        float s2 = warp_sum(v2);
        w = (p.k > 1) ? v2 / (s2 + 1e-20f) : v2;
      } else {
        w = (lane < p.k) ? raw : 0.f;
      }
      w *= p.scaling;
    }
    for (int r = 0; r < p.k; ++r) {
      if (lane == r) {
        const int e_sel = idx[r] < p.E ? idx[r] : p.E - 1;   // k > number of selectable experts: stay in range
        p.topk_idx[t * p.k + r] = e_sel;
        p.topk_prob[t * p.k + r] = w;
        if (p.counts) atomicAdd(&p.counts[e_sel], 1);
      }
    }
    // aux statistics: bias-free top-k over normalised scores, padding excluded
    const bool valid = p.valid_mask ? (p.valid_mask[t] != 0) : true;
    if ((p.score_partial || p.aux_counts) && valid) {
      float nsc[MAX_E_PER_LANE];
      const float inv = (p.score_fn == SIGMOID) ? 1.f / (ssum + 1e-20f) : 1.f;
#pragma unroll
      for (int j = 0; j < MAX_E_PER_LANE; ++j) nsc[j] = (lg[j] == -INFINITY) ? -INFINITY : sc[j] * inv;
      if (p.aux_counts) {
        int aidx[MAX_K];
        if (p.expert_bias) {
          warp_topk(nsc, epl, p.E, p.k, lane, aidx);
        } else {
#pragma unroll
          for (int r = 0; r < MAX_K; ++r) aidx[r] = idx[r];
        }
        for (int r = 0; r < p.k; ++r)
          if (lane == r) atomicAdd(&p.aux_counts[aidx[r] < p.E ? aidx[r] : p.E - 1], 1);
      }
      if (p.score_partial) {
#pragma unroll
        for (int j = 0; j < MAX_E_PER_LANE; ++j) {
          int e = j * 32 + lane;
          if (j < epl && e < p.E) atomicAdd(&s_scores[e], nsc[j]);
        }
      }
    }
  }
  if (p.score_partial) {
    __syncthreads();
    for (int i = threadIdx.x; i < p.E; i += blockDim.x)
      p.score_partial[static_cast<long long>(blockIdx.x) * p.E + i] = s_scores[i];
  }
}

struct RouterBwdParams {
  const float* logits;     // [T, E]
  const int* topk_idx;     // [T, k]
  const float* topk_prob;  // [T, k] forward output (after scaling)
  const float* dprob;      // [T, k] or null
  const float* aux_grad;   // [E] or null: d(loss)/d(aux score of expert e), applied to valid tokens
  const float* lse;        // unused (kept for ABI symmetry with the forward)
  const unsigned char* valid_mask;
  const float* dlse;       // [T] or null: d(loss)/d(lse_t)
  float* dlogits;          // [T, E] fp32
  long long T;
  int E, k, score_fn;
  float scaling;
};

__global__ void router_bwd_kernel(const RouterBwdParams p) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int epl = (p.E + 31) / 32;
  for (long long t = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); t < p.T;
       t += static_cast<long long>(gridDim.x) * wpb) {
    float lg[MAX_E_PER_LANE], sc[MAX_E_PER_LANE], ds[MAX_E_PER_LANE], dl[MAX_E_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      int e = j * 32 + lane;
      lg[j] = (j < epl && e < p.E) ? p.logits[t * p.E + e] : -INFINITY;
      mx = fmaxf(mx, lg[j]);
      ds[j] = 0.f;
      dl[j] = 0.f;
    }
    mx = warp_max(mx);
    float se = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) se += (lg[j] == -INFINITY) ? 0.f : __expf(lg[j] - mx);
    se = warp_sum(se);
    const float lse = mx + logf(se);
    float ssum = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      if (lg[j] == -INFINITY) { sc[j] = 0.f; continue; }
      sc[j] = (p.score_fn == SIGMOID) ? 1.f / (1.f + __expf(-lg[j])) : __expf(lg[j] - lse);
      ssum += sc[j];
    }
    if (p.score_fn == SIGMOID) ssum = warp_sum(ssum);
    const bool valid = p.valid_mask ? (p.valid_mask[t] != 0) : true;

    // ---- routing-weight gradient
    if (p.dprob) {
      // lane r holds (idx_r, w_r, dw_r)
      int my_e = (lane < p.k) ? p.topk_idx[t * p.k + lane] : -1;
      float my_w = (lane < p.k) ? p.topk_prob[t * p.k + lane] / p.scaling : 0.f;  // unscaled weight
      float my_d = (lane < p.k) ? p.dprob[t * p.k + lane] * p.scaling : 0.f;      // grad wrt unscaled weight
      float g_sel = 0.f;  // gradient wrt the selected raw value (logit for POST, score otherwise)
      if (p.score_fn == SOFTMAX_POST) {
        float dot = warp_sum(my_d * my_w);
        g_sel = my_w * (my_d - dot);  // already d(logit)
      } else if (p.score_fn == SIGMOID && p.k > 1) {
        // w_j = s_j / (S + eps): dw/ds_i = (delta_ij - w_j) / (S + eps)
        float S = 0.f;
        {
          float sraw = 0.f;
          for (int r = 0; r < p.k; ++r) {
            int e = __shfl_sync(0xffffffffu, my_e, r);
            float vv = 0.f;
#pragma unroll
            for (int j = 0; j < MAX_E_PER_LANE; ++j)
              if (j == (e >> 5)) vv = sc[j];
            vv = __shfl_sync(0xffffffffu, vv, e & 31);
            if (lane == r) sraw = vv;
          }
          S = warp_sum(sraw) + 1e-20f;
        }
        float dot = warp_sum(my_d * my_w);
        g_sel = (my_d - dot) / S;
      } else {
        g_sel = my_d;
      }
      // scatter g_sel to the owning lane/slot
      for (int r = 0; r < p.k; ++r) {
        int e = __shfl_sync(0xffffffffu, my_e, r);
        float g = __shfl_sync(0xffffffffu, g_sel, r);
        if ((e & 31) == lane) {
#pragma unroll
          for (int j = 0; j < MAX_E_PER_LANE; ++j)
            if (j == (e >> 5)) {
              if (p.score_fn == SOFTMAX_POST) dl[j] += g; else ds[j] += g;
            }
        }
      }
    }
    // ---- aux-loss gradient on normalised scores
    if (p.aux_grad && valid) {
      if (p.score_fn == SIGMOID) {
        // n_e = s_e / (S_all + eps); dn/ds_i = (delta - n_e)/(S_all + eps)
        const float Sall = ssum + 1e-20f;
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < MAX_E_PER_LANE; ++j) {
          int e = j * 32 + lane;
          if (j < epl && e < p.E) dot += p.aux_grad[e] * sc[j] / Sall;
        }
        dot = warp_sum(dot);
#pragma unroll
        for (int j = 0; j < MAX_E_PER_LANE; ++j) {
          int e = j * 32 + lane;
          if (j < epl && e < p.E) ds[j] += (p.aux_grad[e] - dot) / Sall;
        }
      } else {
#pragma unroll
        for (int j = 0; j < MAX_E_PER_LANE; ++j) {
          int e = j * 32 + lane;
          if (j < epl && e < p.E) ds[j] += p.aux_grad[e];
        }
      }
    }
    // ---- score -> logit jacobian
    if (p.score_fn == SIGMOID) {
#pragma unroll
      for (int j = 0; j < MAX_E_PER_LANE; ++j) dl[j] += ds[j] * sc[j] * (1.f - sc[j]);
    } else {
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < MAX_E_PER_LANE; ++j) dot += ds[j] * sc[j];
      dot = warp_sum(dot);
#pragma unroll
      for (int j = 0; j < MAX_E_PER_LANE; ++j) dl[j] += sc[j] * (ds[j] - dot);
    }
    // ---- logsumexp gradient (z-loss): d(lse)/dl = softmax(l)
    if (p.dlse) {
      const float zc = p.dlse[t];
#pragma unroll
      for (int j = 0; j < MAX_E_PER_LANE; ++j)
        if (lg[j] != -INFINITY) dl[j] += zc * __expf(lg[j] - lse);
    }
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      int e = j * 32 + lane;
      if (j < epl && e < p.E) p.dlogits[t * p.E + e] = dl[j];
    }
  }
}

__global__ void colsum_f32_kernel(const float* __restrict__ partial, float* __restrict__ out, int rows, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int r = 0; r < rows; ++r) s += partial[static_cast<long long>(r) * cols + c];
  out[c] = s;
}

// ============================================================================
// Permutation index.  idx: [N] int32 expert ids (N = T*k, token-major).
//   pass 1: counts[e]
//   pass 2: seg_start[E+1] (128-aligned exclusive scan), tile_group[m_tiles_cap],
//           group_rows (== seg_start) and total_rows
//   pass 3: row_of[n] = seg_start[e] + rank of n among entries with expert e (stable)
// ============================================================================
__global__ void perm_count_kernel(const int* __restrict__ idx, long long N, int* __restrict__ counts) {
  __shared__ int red[32];
  const int e = blockIdx.x;
  int c = 0;
  for (long long i = threadIdx.x; i < N; i += blockDim.x) c += (idx[i] == e);
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x < 32) {
    int v = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) counts[e] = v;
  }
}

__global__ void perm_scan_kernel(const int* __restrict__ counts, int E, int* __restrict__ seg_start,
                                 int* __restrict__ tile_group, int m_tiles_cap, int* __restrict__ status) {
  // single block; E <= 1024
  __shared__ int s_start[1025];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_start[e] = acc;
      acc += ((counts[e] + SEG_ALIGN - 1) / SEG_ALIGN) * SEG_ALIGN;
    }
    s_start[E] = acc;
    if (acc > m_tiles_cap * SEG_ALIGN && status) status[0] = 1;  // capacity exceeded
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= E; i += blockDim.x) seg_start[i] = s_start[i];
  for (int m = threadIdx.x; m < m_tiles_cap; m += blockDim.x) {
    const int row = m * SEG_ALIGN;
    int g = -1;
    if (row < s_start[E]) {
      int lo = 0, hi = E;  // find e with s_start[e] <= row < s_start[e+1]
      while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (s_start[mid] <= row) lo = mid; else hi = mid;
      }
      g = lo;
    }
    tile_group[m] = g;
  }
}

__global__ void perm_rank_kernel(const int* __restrict__ idx, long long N, const int* __restrict__ seg_start,
                                 int* __restrict__ row_of, const int* __restrict__ order_base, int* __restrict__ order) {
  // `order` (optional): the inverse of a second packing of the same entries, order[order_base[e] + rank] = entry
  __shared__ int warp_tot[32];
  __shared__ int base, obase;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (threadIdx.x == 0) {
    base = seg_start[e];
    obase = order ? order_base[e] : 0;
  }
  __syncthreads();
  for (long long i0 = 0; i0 < N; i0 += blockDim.x) {
    const long long i = i0 + threadIdx.x;
    const bool hit = (i < N) && (idx[i] == e);
    const unsigned bal = __ballot_sync(0xffffffffu, hit);
    const int pre = __popc(bal & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[w] = __popc(bal);
    __syncthreads();
    int woff = 0, tot = 0;
    for (int j = 0; j < nw; ++j) {
      int v = warp_tot[j];
      if (j < w) woff += v;
      tot += v;
    }
    if (hit) {
      row_of[i] = base + woff + pre;
      if (order) order[obase + woff + pre] = static_cast<int>(i);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      base += tot;
      obase += tot;
    }
    __syncthreads();
  }
}

// dst[row_of[n], :] = src[n / k, :]; row_val_out[row_of[n]] = val[n] (optional).  One warp per entry.
__global__ void perm_scatter_kernel(const __nv_bfloat16* __restrict__ src, long long lds,
                                    __nv_bfloat16* __restrict__ dst, long long ldd, const int* __restrict__ row_of,
                                    const float* __restrict__ val, float* __restrict__ row_val_out,
                                    int* __restrict__ row_src_out, long long N, int k, int H) {
  const long long n = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (n >= N) return;
  const long long t = n / k;
  const long long r = row_of[n];
  const uint4* s = reinterpret_cast<const uint4*>(src + t * lds);
  uint4* d = reinterpret_cast<uint4*>(dst + r * ldd);
  for (int c = lane; c < H / 8; c += 32) d[c] = s[c];
  if (lane == 0) {
    if (row_val_out) row_val_out[r] = val[n];
    if (row_src_out) row_src_out[r] = static_cast<int>(n);
  }
}

// zero the pad rows [seg_start[e] + counts[e], seg_start[e+1]) of every expert (their scalars become 0, their return
// tags -1); `zero_ints` (optional, `n_zero` entries) is cleared as well: the progress counters of the next exchange
__global__ void perm_zero_pad_kernel(__nv_bfloat16* __restrict__ dst, long long ldd, const int* __restrict__ counts,
                                     const int* __restrict__ seg_start, float* __restrict__ row_val_out,
                                     int* __restrict__ row_tag_out, int* __restrict__ zero_ints, int n_zero, int H) {
  const int e = blockIdx.x;
  const int r0 = seg_start[e] + counts[e], r1 = seg_start[e + 1];
  const uint4 z = make_uint4(0, 0, 0, 0);
  const int vec = H / 8;
  for (long long i = threadIdx.x; i < static_cast<long long>(r1 - r0) * vec; i += blockDim.x) {
    const long long r = r0 + i / vec;
    reinterpret_cast<uint4*>(dst + r * ldd)[i % vec] = z;
  }
  for (int r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
    if (row_val_out) row_val_out[r] = 0.f;
    if (row_tag_out) row_tag_out[r] = -1;
  }
  if (zero_ints)
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_zero; i += gridDim.x * blockDim.x) zero_ints[i] = 0;
}

// out[t, :] = sum_j w[t,j] * src[row_of[t*k + j], :] (+ residual[t, :]).  One block per token.
__global__ void perm_combine_kernel(const __nv_bfloat16* __restrict__ src, long long lds,
                                    const int* __restrict__ row_of, const float* __restrict__ w,
                                    const __nv_bfloat16* __restrict__ residual, long long ldr,
                                    __nv_bfloat16* __restrict__ out, long long ldo, int k, int H) {
  const long long t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const long long r = row_of[t * k + j];
      const float wt = w ? w[t * k + j] : 1.f;
      uint4 u = *reinterpret_cast<const uint4*>(src + r * lds + c);
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += wt * a.x; acc[1] += wt * a.y; acc[2] += wt * b.x; acc[3] += wt * b.y;
      acc[4] += wt * cc.x; acc[5] += wt * cc.y; acc[6] += wt * d.x; acc[7] += wt * d.y;
    }
    if (residual) {
      uint4 u = *reinterpret_cast<const uint4*>(residual + t * ldr + c);
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + t * ldo + c) = o;
  }
}


// ------------------------------------------------------------------------------------------------------------
// Load-balance (auxiliary) loss of one router from the statistics the routing kernel already produced:
//   aux = scale_num * sum_e score_sum[e] * cnt[e] / (k * n^2),   n = max(sum_e cnt[e] / k, 1)
// out[0] = aux, out[1] = aux / coeff (the unscaled value for logging); coef[e] = d aux / d score_sum[e].
// One block.  Replaces a chain of a dozen elementwise / reduction launches per MoE layer
// (models/modules/moe/router.py:164-200 of the reference computes the same quantity with torch ops).
// ------------------------------------------------------------------------------------------------------------
__global__ void aux_loss_kernel(const float* __restrict__ score_sum, const int* __restrict__ cnt, int E, int k,
                                float scale_num, float coeff, float* __restrict__ out, float* __restrict__ coef) {
  __shared__ float red[32];
  __shared__ float s_n, s_dot;
  float c = 0.f, d = 0.f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float ce = static_cast<float>(cnt[e]);
    c += ce;
    d += score_sum[e] * ce;
  }
  c = warp_sum(c);
  d = warp_sum(d);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red[w] = c;
  __syncthreads();
  if (w == 0) {
    float t = l < nw ? red[l] : 0.f;
    t = warp_sum(t);
    if (l == 0) s_n = fmaxf(t / static_cast<float>(k), 1.f);
  }
  __syncthreads();
  if (l == 0) red[w] = d;
  __syncthreads();
  if (w == 0) {
    float t = l < nw ? red[l] : 0.f;
    t = warp_sum(t);
    if (l == 0) s_dot = t;
  }
  __syncthreads();
  const float f = scale_num / (static_cast<float>(k) * s_n * s_n);
  if (threadIdx.x == 0) {
    out[0] = s_dot * f;
    out[1] = coeff != 0.f ? s_dot * f / coeff : 0.f;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) coef[e] = static_cast<float>(cnt[e]) * f;
}

}  // namespace ttb

using namespace ttb;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_RET() do { cudaError_t e__ = cudaGetLastError(); return e__ == cudaSuccess ? 0 : 400 + (int)e__; } while (0)

// score_partial: [grid, E] scratch; score_sum: [E] output (may be null together with score_partial)
TTB_EXPORT int ttb_router_fwd(const float* logits, const float* expert_bias, const unsigned char* valid_mask,
                              int* topk_idx, float* topk_prob, float* lse, float* score_partial, float* score_sum,
                              int* aux_counts, int* counts, long long T, int E, int k, int score_fn, float scaling,
                              int grid, void* stream) {
  if (E > 32 * MAX_E_PER_LANE || k > MAX_K || k > E || k > 32) return 901;
  if (T == 0) return 0;
  RouterParams p{logits, expert_bias, valid_mask, topk_idx, topk_prob, lse, score_partial, aux_counts, counts, T, E, k,
                 score_fn, scaling};
  const long long need = (T + 7) / 8;
  if (grid > need) grid = (int)need;
  router_fwd_kernel<<<grid, 256, E * sizeof(float), STREAM(stream)>>>(p);
  if (score_partial && score_sum)
    colsum_f32_kernel<<<(E + 127) / 128, 128, 0, STREAM(stream)>>>(score_partial, score_sum, grid, E);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_router_bwd(const float* logits, const int* topk_idx, const float* topk_prob, const float* dprob,
                              const float* aux_grad, const float* lse, const unsigned char* valid_mask,
                              const float* dlse, float* dlogits, long long T, int E, int k, int score_fn,
                              float scaling, void* stream) {
  if (E > 32 * MAX_E_PER_LANE || k > MAX_K || k > 32) return 901;
  if (T == 0) return 0;
  RouterBwdParams p{logits, topk_idx, topk_prob, dprob, aux_grad, lse, valid_mask, dlse, dlogits, T, E, k, score_fn,
                    scaling};
  long long grid = (T + 7) / 8;
  if (grid > 4096) grid = 4096;
  router_bwd_kernel<<<(unsigned)grid, 256, 0, STREAM(stream)>>>(p);
  LAUNCH_RET();
}

// Builds the padded (expert, token)-ordered permutation of idx[N].
// counts[E], seg_start[E+1], tile_group[m_tiles_cap], row_of[N], status[1] (set to 1 when capacity is exceeded).
TTB_EXPORT int ttb_perm_index(const int* idx, long long N, int E, int* counts, int* seg_start, int* tile_group,
                              int m_tiles_cap, int* row_of, int* status, void* stream) {
  if (E > 1024) return 901;
  perm_count_kernel<<<E, 256, 0, STREAM(stream)>>>(idx, N, counts);
  perm_scan_kernel<<<1, 256, 0, STREAM(stream)>>>(counts, E, seg_start, tile_group, m_tiles_cap, status);
  perm_rank_kernel<<<E, 256, 0, STREAM(stream)>>>(idx, N, seg_start, row_of, nullptr, nullptr);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_perm_scatter(const void* src, long long lds, void* dst, long long ldd, const int* row_of,
                                const float* val, float* row_val_out, int* row_src_out, const int* counts,
                                const int* seg_start, int E, long long N, int k, int H, void* stream) {
  if (H % 8 || lds % 8 || ldd % 8) return 901;
  if (counts) perm_zero_pad_kernel<<<E, 256, 0, STREAM(stream)>>>((__nv_bfloat16*)dst, ldd, counts, seg_start, row_val_out, nullptr, nullptr, 0, H);
  if (N > 0) {
    const long long blocks = (N + 7) / 8;
    perm_scatter_kernel<<<(unsigned)blocks, 256, 0, STREAM(stream)>>>((const __nv_bfloat16*)src, lds,
                                                                     (__nv_bfloat16*)dst, ldd, row_of, val,
                                                                     row_val_out, row_src_out, N, k, H);
  }
  LAUNCH_RET();
}

TTB_EXPORT int ttb_perm_combine(const void* src, long long lds, const int* row_of, const float* w, const void* residual,
                                long long ldr, void* out, long long ldo, long long T, int k, int H, void* stream) {
  if (H % 8 || lds % 8 || ldo % 8) return 901;
  if (T == 0) return 0;
  int threads = H / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  perm_combine_kernel<<<(unsigned)T, threads, 0, STREAM(stream)>>>((const __nv_bfloat16*)src, lds, row_of, w,
                                                                  (const __nv_bfloat16*)residual, ldr,
                                                                  (__nv_bfloat16*)out, ldo, k, H);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_aux_loss(const float* score_sum, const int* cnt, int E, int k, float scale_num, float coeff, float* out2,
                            float* coef, void* stream) {
  if (E < 1 || k < 1) return 901;
  aux_loss_kernel<<<1, 256, 0, STREAM(stream)>>>(score_sum, cnt, E, k, scale_num, coeff, out2, coef);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_moe_seg_align() { return SEG_ALIGN; }

// row_of[n] = base[idx[n]] + stable rank of n among the entries of its expert (base need not be a scan of counts)
TTB_EXPORT int ttb_perm_rank(const int* idx, long long N, int E, const int* base, int* row_of, void* stream) {
  if (N == 0) return 0;
  perm_rank_kernel<<<E, 256, 0, STREAM(stream)>>>(idx, N, base, row_of, nullptr, nullptr);
  LAUNCH_RET();
}

// same, plus order[order_base[idx[n]] + rank] = n : the entries listed in a second (send) order
TTB_EXPORT int ttb_perm_rank_order(const int* idx, long long N, int E, const int* base, int* row_of, const int* order_base,
                                   int* order, void* stream) {
  if (N == 0) return 0;
  perm_rank_kernel<<<E, 256, 0, STREAM(stream)>>>(idx, N, base, row_of, order_base, order);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_perm_zero_pad(void* dst, long long ldd, const int* counts, const int* seg_start, float* row_val,
                                 int E, int H, void* stream) {
  if (H % 8 || ldd % 8) return 901;
  perm_zero_pad_kernel<<<E, 256, 0, STREAM(stream)>>>((__nv_bfloat16*)dst, ldd, counts, seg_start, row_val, nullptr, nullptr, 0, H);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_perm_zero_pad_tags(void* dst, long long ldd, const int* counts, const int* seg_start, float* row_val,
                                      int* row_tag, int* zero_ints, int n_zero, int E, int H, void* stream) {
  if (H % 8 || ldd % 8) return 901;
  perm_zero_pad_kernel<<<E, 256, 0, STREAM(stream)>>>((__nv_bfloat16*)dst, ldd, counts, seg_start, row_val, row_tag, zero_ints,
                                                     n_zero, H);
  LAUNCH_RET();
}
