// Bandwidth-bound training kernels for sm_100a: RMSNorm (+residual) fwd/bwd,
// fused QK-RMSNorm + rotary embedding fwd/bwd, SwiGLU fwd/bwd (with routing-prob
// scaling), cross-entropy with in-place gradient, multi-tensor AdamW with a
// device-side clip coefficient and multi-tensor squared-norm partials.
//
// Numerical contracts follow the reference's torch formulas:
//   RMSNorm   : fp32 x*rsqrt(mean(x^2)+eps) -> cast -> * weight        (ops/providers/native/rms_norm.py:16-22)
//   SwiGLU    : silu(gate) * up on [gate|up] halves, prob applied after the
//               activation                                             (ops/providers/native/swiglu.py:10-12,
//                                                                       models/modules/moe/experts.py:181-186)
//   CE        : fp32, reduction=sum, ignore_index=-100                (ops/providers/native/cross_entropy_loss.py:17-33)
//   AdamW     : torch fused AdamW math on fp32 shards                  (engine/backends/fsdp2/optimizers/adamw.py:226-251)
#include "common.cuh"

namespace ttb {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : -INFINITY;
  t = warp_max(t);
  __syncthreads();
  return t;
}

// ============================================================================
// RMSNorm forward.  y = bf16(bf16(x_sum * rstd) * w),  x_sum = x (+ residual).
// One block per row, 8 bf16 per thread per iteration (H % 8 == 0).
// ============================================================================
template <int MAX_ITERS>
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd_out, int H, float eps,
                                   int one_plus_w) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  const __nv_bfloat16* rr = residual ? residual + row * H : nullptr;
  float vals[MAX_ITERS][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < MAX_ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c >= H) break;
    uint4 u = *reinterpret_cast<const uint4*>(xr + c);
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
    float f[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
    if (rr) {
      uint4 r = *reinterpret_cast<const uint4*>(rr + c);
      float2 ra = unpack_bf16(r.x), rb = unpack_bf16(r.y), rc = unpack_bf16(r.z), rd = unpack_bf16(r.w);
      float g[8] = {ra.x, ra.y, rb.x, rb.y, rc.x, rc.y, rd.x, rd.y};
      uint4 o;
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(__float2bfloat16(f[j] + g[j]));
      o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]); o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
      *reinterpret_cast<uint4*>(sum_out + row * H + c) = o;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      vals[it][j] = f[j];
      ss += f[j] * f[j];
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / static_cast<float>(H) + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int it = 0; it < MAX_ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c >= H) break;
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = vals[it][j];
    uint4 wu = *reinterpret_cast<const uint4*>(w + c);
    float2 wa = unpack_bf16(wu.x), wb = unpack_bf16(wu.y), wc = unpack_bf16(wu.z), wd = unpack_bf16(wu.w);
    float wf[8] = {wa.x, wa.y, wb.x, wb.y, wc.x, wc.y, wd.x, wd.y};
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float xh = __bfloat162float(__float2bfloat16(f[j] * rstd));
      o[j] = xh * (one_plus_w ? 1.f + wf[j] : wf[j]);
    }
    uint4 ou;
    ou.x = pack_bf16(o[0], o[1]); ou.y = pack_bf16(o[2], o[3]); ou.z = pack_bf16(o[4], o[5]); ou.w = pack_bf16(o[6], o[7]);
    *reinterpret_cast<uint4*>(y + row * H + c) = ou;
  }
}

// RMSNorm backward.  Persistent blocks loop over rows; per-thread dw partials live in
// registers and are flushed to dw_partial[blockIdx.x][H] at the end.
//   dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * w,  xhat = x * rstd   (+ dres_in)
template <int MAX_ITERS>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                                   const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw_partial, long long T, int H, int one_plus_w) {
  __shared__ float red[32];
  float dwacc[MAX_ITERS][8];
#pragma unroll
  for (int i = 0; i < MAX_ITERS; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float xh[MAX_ITERS][8], g[MAX_ITERS][8];
    float dot = 0.f;
#pragma unroll
    for (int it = 0; it < MAX_ITERS; ++it) {
      const int c = (it * blockDim.x + threadIdx.x) * 8;
      if (c >= H) break;
      uint4 xu = *reinterpret_cast<const uint4*>(x + row * H + c);
      uint4 du = *reinterpret_cast<const uint4*>(dy + row * H + c);
      uint4 wu = *reinterpret_cast<const uint4*>(w + c);
      uint32_t xs[4] = {xu.x, xu.y, xu.z, xu.w}, ds[4] = {du.x, du.y, du.z, du.w}, ws[4] = {wu.x, wu.y, wu.z, wu.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 xf = unpack_bf16(xs[j]), df = unpack_bf16(ds[j]), wf = unpack_bf16(ws[j]);
        if (one_plus_w) { wf.x += 1.f; wf.y += 1.f; }
        float h0 = xf.x * rstd, h1 = xf.y * rstd;
        xh[it][2 * j] = h0; xh[it][2 * j + 1] = h1;
        g[it][2 * j] = df.x * wf.x; g[it][2 * j + 1] = df.y * wf.y;
        dot += g[it][2 * j] * h0 + g[it][2 * j + 1] * h1;
        dwacc[it][2 * j] += df.x * h0;
        dwacc[it][2 * j + 1] += df.y * h1;
      }
    }
    dot = block_sum(dot, red) / static_cast<float>(H);
#pragma unroll
    for (int it = 0; it < MAX_ITERS; ++it) {
      const int c = (it * blockDim.x + threadIdx.x) * 8;
      if (c >= H) break;
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * (g[it][j] - xh[it][j] * dot);
      if (dres_in) {
        uint4 r = *reinterpret_cast<const uint4*>(dres_in + row * H + c);
        float2 a = unpack_bf16(r.x), b = unpack_bf16(r.y), cc = unpack_bf16(r.z), d = unpack_bf16(r.w);
        o[0] += a.x; o[1] += a.y; o[2] += b.x; o[3] += b.y; o[4] += cc.x; o[5] += cc.y; o[6] += d.x; o[7] += d.y;
      }
      uint4 ou;
      ou.x = pack_bf16(o[0], o[1]); ou.y = pack_bf16(o[2], o[3]); ou.z = pack_bf16(o[4], o[5]); ou.w = pack_bf16(o[6], o[7]);
      *reinterpret_cast<uint4*>(dx + row * H + c) = ou;
    }
  }
#pragma unroll
  for (int it = 0; it < MAX_ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c >= H) break;
    float* dst = dw_partial + static_cast<long long>(blockIdx.x) * H + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = dwacc[it][j];
  }
}

// Column sum of partial[rows][H] -> out[H] (fp32); deterministic order.
__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int rows, int H) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int r = 0; r < rows; ++r) s += partial[static_cast<long long>(r) * H + c];
  out[c] = s;
}

// ============================================================================
// LayerNorm (weight + bias) for the vision tower: fp32 statistics, bf16 in / out.
//   y = (x - mean) * rstd * w + b
//   dx = rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dy * w ; dw = sum dy * xhat ; db = sum dy
// Forward: one block per row.  Backward: persistent blocks, per-thread dw / db partials flushed to
// part[blockIdx.x][2][H] and reduced by colsum_kernel (deterministic order).
// HF ViT eager `nn.LayerNorm` of the reference's vision blocks (models/qwen3_5/modeling_qwen3_5.py:1035-1207).
// ============================================================================
template <int MAX_ITERS>
__global__ void layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                     const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                     float* __restrict__ mean_out, float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  float vals[MAX_ITERS][8];
  float s = 0.f;
#pragma unroll
  for (int it = 0; it < MAX_ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) vals[it][j] = 0.f;
    if (c >= H) continue;
    const uint4 u = *reinterpret_cast<const uint4*>(x + row * H + c);
    const float2 a = unpack_bf16(u.x), bb = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
    vals[it][0] = a.x; vals[it][1] = a.y; vals[it][2] = bb.x; vals[it][3] = bb.y;
    vals[it][4] = cc.x; vals[it][5] = cc.y; vals[it][6] = d.x; vals[it][7] = d.y;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += vals[it][j];
  }
  const float mean = block_sum(s, red) / static_cast<float>(H);
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < MAX_ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c >= H) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float d = vals[it][j] - mean;
      ss += d * d;
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / static_cast<float>(H) + eps);
  if (threadIdx.x == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int it = 0; it < MAX_ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c >= H) continue;
    const uint4 wu = *reinterpret_cast<const uint4*>(w + c);
    const uint4 bu = *reinterpret_cast<const uint4*>(b + c);
    const uint32_t ws[4] = {wu.x, wu.y, wu.z, wu.w}, bs[4] = {bu.x, bu.y, bu.z, bu.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 wf = unpack_bf16(ws[j]), bf = unpack_bf16(bs[j]);
      o[j] = pack_bf16((vals[it][2 * j] - mean) * rstd * wf.x + bf.x, (vals[it][2 * j + 1] - mean) * rstd * wf.y + bf.y);
    }
    *reinterpret_cast<uint4*>(y + row * H + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int MAX_ITERS>
__global__ void layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                     const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                                     const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                                     float* __restrict__ part, long long T, int H) {
  __shared__ float red[32];
  float dwacc[MAX_ITERS][8], dbacc[MAX_ITERS][8];
#pragma unroll
  for (int i = 0; i < MAX_ITERS; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { dwacc[i][j] = 0.f; dbacc[i][j] = 0.f; }
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[MAX_ITERS][8], g[MAX_ITERS][8];
    float sg = 0.f, sgx = 0.f;
#pragma unroll
    for (int it = 0; it < MAX_ITERS; ++it) {
      const int c = (it * blockDim.x + threadIdx.x) * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) { xh[it][j] = 0.f; g[it][j] = 0.f; }
      if (c >= H) continue;
      const uint4 xu = *reinterpret_cast<const uint4*>(x + row * H + c);
      const uint4 du = *reinterpret_cast<const uint4*>(dy + row * H + c);
      const uint4 wu = *reinterpret_cast<const uint4*>(w + c);
      const uint32_t xs[4] = {xu.x, xu.y, xu.z, xu.w}, ds[4] = {du.x, du.y, du.z, du.w}, ws[4] = {wu.x, wu.y, wu.z, wu.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = unpack_bf16(xs[j]), df = unpack_bf16(ds[j]), wf = unpack_bf16(ws[j]);
        const float h0 = (xf.x - mean) * rstd, h1 = (xf.y - mean) * rstd;
        xh[it][2 * j] = h0; xh[it][2 * j + 1] = h1;
        g[it][2 * j] = df.x * wf.x; g[it][2 * j + 1] = df.y * wf.y;
        sg += g[it][2 * j] + g[it][2 * j + 1];
        sgx += g[it][2 * j] * h0 + g[it][2 * j + 1] * h1;
        dwacc[it][2 * j] += df.x * h0; dwacc[it][2 * j + 1] += df.y * h1;
        dbacc[it][2 * j] += df.x; dbacc[it][2 * j + 1] += df.y;
      }
    }
    sg = block_sum(sg, red) / static_cast<float>(H);
    sgx = block_sum(sgx, red) / static_cast<float>(H);
#pragma unroll
    for (int it = 0; it < MAX_ITERS; ++it) {
      const int c = (it * blockDim.x + threadIdx.x) * 8;
      if (c >= H) continue;
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = pack_bf16(rstd * (g[it][2 * j] - sg - xh[it][2 * j] * sgx), rstd * (g[it][2 * j + 1] - sg - xh[it][2 * j + 1] * sgx));
      *reinterpret_cast<uint4*>(dx + row * H + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
#pragma unroll
  for (int it = 0; it < MAX_ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c >= H) continue;
    float* dwp = part + static_cast<long long>(blockIdx.x) * 2 * H + c;
    float* dbp = dwp + H;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dwp[j] = dwacc[it][j]; dbp[j] = dbacc[it][j]; }
  }
}

// ============================================================================
// y = act(x + bias) (+ residual): the elementwise tail of a biased projection in one pass.
//   act 0: identity, 1: GELU (tanh approximation), 2: GELU (erf).   x [R, C], bias [C], residual [R, C]; C % 8 == 0
// Backward: dx = dy * act'(x + bias) ; dbias = column sum of dx (partials per block, reduced by colsum_kernel).
// ============================================================================
__device__ __forceinline__ float act_fwd(float v, int act) {
  if (act == 1) {
    const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.f + tanhf(u));
  }
  if (act == 2) return 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
  return v;
}
__device__ __forceinline__ float act_grad(float v, int act) {
  if (act == 1) {
    const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    const float t = tanhf(u);
    return 0.5f * (1.f + t) + 0.5f * v * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * v * v);
  }
  if (act == 2) return 0.5f * (1.f + erff(v * 0.7071067811865476f)) + v * 0.3989422804014327f * __expf(-0.5f * v * v);
  return 1.f;
}

__global__ void bias_act_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias,
                                    const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ y,
                                    long long R, int C, int act) {
  const long long vec_per_row = C / 8;
  const long long total = R * vec_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const uint4 xu = *(reinterpret_cast<const uint4*>(x) + i);
    const uint4 bu = *reinterpret_cast<const uint4*>(bias + c);
    uint4 ru = make_uint4(0u, 0u, 0u, 0u);
    if (residual) ru = *(reinterpret_cast<const uint4*>(residual) + i);
    const uint32_t xs[4] = {xu.x, xu.y, xu.z, xu.w}, bs[4] = {bu.x, bu.y, bu.z, bu.w}, rs[4] = {ru.x, ru.y, ru.z, ru.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xf = unpack_bf16(xs[j]), bf = unpack_bf16(bs[j]), rf = unpack_bf16(rs[j]);
      o[j] = pack_bf16(act_fwd(xf.x + bf.x, act) + rf.x, act_fwd(xf.y + bf.y, act) + rf.y);
    }
    *(reinterpret_cast<uint4*>(y) + i) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int MAX_ITERS>
__global__ void bias_act_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                    const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ dx,
                                    float* __restrict__ part, long long R, int C, int act) {
  float acc[MAX_ITERS][8];
#pragma unroll
  for (int i = 0; i < MAX_ITERS; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  for (long long row = blockIdx.x; row < R; row += gridDim.x) {
#pragma unroll
    for (int it = 0; it < MAX_ITERS; ++it) {
      const int c = (it * blockDim.x + threadIdx.x) * 8;
      if (c >= C) continue;
      const uint4 du = *reinterpret_cast<const uint4*>(dy + row * C + c);
      const uint32_t ds[4] = {du.x, du.y, du.z, du.w};
      uint32_t o[4];
      if (act == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 df = unpack_bf16(ds[j]);
          acc[it][2 * j] += df.x; acc[it][2 * j + 1] += df.y;
          o[j] = ds[j];
        }
      } else {
        const uint4 xu = *reinterpret_cast<const uint4*>(x + row * C + c);
        const uint4 bu = *reinterpret_cast<const uint4*>(bias + c);
        const uint32_t xs[4] = {xu.x, xu.y, xu.z, xu.w}, bs[4] = {bu.x, bu.y, bu.z, bu.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 df = unpack_bf16(ds[j]), xf = unpack_bf16(xs[j]), bf = unpack_bf16(bs[j]);
          const float g0 = df.x * act_grad(xf.x + bf.x, act), g1 = df.y * act_grad(xf.y + bf.y, act);
          acc[it][2 * j] += g0; acc[it][2 * j + 1] += g1;
          o[j] = pack_bf16(g0, g1);
        }
      }
      if (dx) *reinterpret_cast<uint4*>(dx + row * C + c) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
#pragma unroll
  for (int it = 0; it < MAX_ITERS; ++it) {
    const int c = (it * blockDim.x + threadIdx.x) * 8;
    if (c >= C) continue;
    float* dst = part + static_cast<long long>(blockIdx.x) * C + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = acc[it][j];
  }
}

// ============================================================================
// Causal depthwise short convolution over a packed row (linear-attention mixers: GDN / KDA q, k, v streams).
//   pre[t, c] = bias[c] + sum_{s < W} w[c, W-1-s] * x[t-s, c]   for t-s inside t's sequence;   y = silu(pre) or pre
// x, y: [T, D] bf16 (D % 8 == 0), w: [D, W] bf16 (tap W-1 multiplies the current token), seq_start[t] = first token of
// t's sequence, seq_end[t] = one past its last.  W <= 8.
// Backward: dpre = dy * act'(pre) (pre is recomputed);  dx[t] = sum_s w[., W-1-s] * dpre[t+s] for t+s in the sequence;
// dw[c, W-1-s] = sum_t dpre[t, c] * x[t-s, c];  db = sum_t dpre.  Pass 1 writes dpre (bf16) and per-block dw / db
// partials; pass 2 forms dx.  Torch formulation: ops/providers/native/causal_conv1d.py of the reference (fla Triton
// kernel on its GPU path).
// ============================================================================
constexpr int CONV_MAX_W = 8;   // widest supported filter (kernels are instantiated for <= 4 and <= 8 taps)

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}

// grid: (ceil(D/8 / blockDim.x), row blocks); each thread owns 8 channels and walks rows [r0, r1)
template <bool BWD, int WMAX>
__global__ void causal_conv1d_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                     const __nv_bfloat16* __restrict__ bias, const int* __restrict__ seq_start,
                                     const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ out,
                                     float* __restrict__ part, long long T, int D, int W, int silu, int rows_per_block) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= D) return;
  float wt[WMAX][8];   // wt[s] = tap for distance s into the past
#pragma unroll
  for (int s = 0; s < WMAX; ++s)
#pragma unroll
    for (int j = 0; j < 8; ++j) wt[s][j] = (s < W) ? __bfloat162float(w[static_cast<long long>(c + j) * W + (W - 1 - s)]) : 0.f;
  float bs[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) bs[j] = bias ? __bfloat162float(bias[c + j]) : 0.f;
  float dwacc[WMAX][8], dbacc[8];
  if (BWD) {
#pragma unroll
    for (int s = 0; s < WMAX; ++s)
#pragma unroll
      for (int j = 0; j < 8; ++j) dwacc[s][j] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) dbacc[j] = 0.f;
  }
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_block;
  const long long r1 = (r0 + rows_per_block < T) ? r0 + rows_per_block : T;
  for (long long t = r0; t < r1; ++t) {
    const long long first = seq_start[t];
    float xs[WMAX][8];
    float pre[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) pre[j] = bs[j];
#pragma unroll
    for (int s = 0; s < WMAX; ++s) {
      if (s < W && t - s >= first) {
        load8(x + (t - s) * D + c, xs[s]);
#pragma unroll
        for (int j = 0; j < 8; ++j) pre[j] += wt[s][j] * xs[s][j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) xs[s][j] = 0.f;
      }
    }
    float o[8];
    if (!BWD) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = silu ? pre[j] / (1.f + __expf(-pre[j])) : pre[j];
    } else {
      float g[8];
      load8(dy + t * D + c, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float d = g[j];
        if (silu) {
          const float sg = 1.f / (1.f + __expf(-pre[j]));
          d *= sg * (1.f + pre[j] * (1.f - sg));
        }
        o[j] = d;
        dbacc[j] += d;
#pragma unroll
        for (int s = 0; s < WMAX; ++s) dwacc[s][j] += d * xs[s][j];
      }
    }
    store8(out + t * D + c, o);
  }
  if (BWD) {
    // part[blockIdx.y][(W + 1)][D]: W tap planes (distance s) then the bias plane
    float* base = part + static_cast<long long>(blockIdx.y) * (W + 1) * D;
#pragma unroll
    for (int s = 0; s < WMAX; ++s)
      if (s < W)
#pragma unroll
        for (int j = 0; j < 8; ++j) base[static_cast<long long>(s) * D + c + j] = dwacc[s][j];
#pragma unroll
    for (int j = 0; j < 8; ++j) base[static_cast<long long>(W) * D + c + j] = dbacc[j];
  }
}

// dx[t] = sum_s w[., W-1-s] * dpre[t+s] for t+s < seq_end[t]
template <int WMAX>
__global__ void causal_conv1d_dx_kernel(const __nv_bfloat16* __restrict__ dpre, const __nv_bfloat16* __restrict__ w,
                                        const int* __restrict__ seq_end, __nv_bfloat16* __restrict__ dx, long long T,
                                        int D, int W, int rows_per_block) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= D) return;
  float wt[WMAX][8];
#pragma unroll
  for (int s = 0; s < WMAX; ++s)
#pragma unroll
    for (int j = 0; j < 8; ++j) wt[s][j] = (s < W) ? __bfloat162float(w[static_cast<long long>(c + j) * W + (W - 1 - s)]) : 0.f;
  const long long r0 = static_cast<long long>(blockIdx.y) * rows_per_block;
  const long long r1 = (r0 + rows_per_block < T) ? r0 + rows_per_block : T;
  for (long long t = r0; t < r1; ++t) {
    const long long last = seq_end[t];
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int s = 0; s < WMAX; ++s) {
      if (s < W && t + s < last) {
        float g[8];
        load8(dpre + (t + s) * D + c, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += wt[s][j] * g[j];
      }
    }
    store8(dx + t * D + c, acc);
  }
}

// ============================================================================
// Fused per-head RMSNorm + rotary embedding (half rotation) for q and k.
// in : qkv [T, ld] bf16 with q heads at column 0, k heads at column Hq*D
// out: q_out [T, Hq, D], k_out [T, Hk, D]  (v is consumed in place by attention)
// cos/sin: [T, D/2] fp32.  One warp per (token, head); D == 128.
// ============================================================================
__global__ void qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld, int Hq, int Hk,
                                       const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                                       const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                       __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                                       float* __restrict__ rstd_out, long long T, float eps, int use_norm) {
  constexpr int D = 128;
  const int lane = threadIdx.x & 31;
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int heads = Hq + Hk;
  if (gw >= T * heads) return;
  const long long t = gw / heads;
  const int h = static_cast<int>(gw - t * heads);
  const bool is_q = h < Hq;
  const __nv_bfloat16* src = qkv + t * ld + static_cast<long long>(h) * D;
  const __nv_bfloat16* w = is_q ? wq : wk;
  __nv_bfloat16* dst = is_q ? q_out + (t * Hq + h) * D : k_out + (t * Hk + (h - Hq)) * D;
  // lane owns columns {2l, 2l+1} and {64+2l, 64+2l+1}
  float2 lo = unpack_bf16(*reinterpret_cast<const uint32_t*>(src + 2 * lane));
  float2 hi = unpack_bf16(*reinterpret_cast<const uint32_t*>(src + 64 + 2 * lane));
  float rstd = 1.f;
  if (use_norm) {
    float ss = lo.x * lo.x + lo.y * lo.y + hi.x * hi.x + hi.y * hi.y;
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / D + eps);
    float2 wl = unpack_bf16(*reinterpret_cast<const uint32_t*>(w + 2 * lane));
    float2 wh = unpack_bf16(*reinterpret_cast<const uint32_t*>(w + 64 + 2 * lane));
    lo.x = __bfloat162float(__float2bfloat16(lo.x * rstd)) * wl.x;
    lo.y = __bfloat162float(__float2bfloat16(lo.y * rstd)) * wl.y;
    hi.x = __bfloat162float(__float2bfloat16(hi.x * rstd)) * wh.x;
    hi.y = __bfloat162float(__float2bfloat16(hi.y * rstd)) * wh.y;
    // the normalised tensor is a bf16 tensor in the eager formulation
    lo.x = __bfloat162float(__float2bfloat16(lo.x)); lo.y = __bfloat162float(__float2bfloat16(lo.y));
    hi.x = __bfloat162float(__float2bfloat16(hi.x)); hi.y = __bfloat162float(__float2bfloat16(hi.y));
  }
  if (rstd_out && lane == 0) rstd_out[gw] = rstd;
  const float2 c = *reinterpret_cast<const float2*>(cos_t + t * (D / 2) + 2 * lane);
  const float2 s = *reinterpret_cast<const float2*>(sin_t + t * (D / 2) + 2 * lane);
  float o_lo_x = lo.x * c.x - hi.x * s.x, o_lo_y = lo.y * c.y - hi.y * s.y;
  float o_hi_x = hi.x * c.x + lo.x * s.x, o_hi_y = hi.y * c.y + lo.y * s.y;
  *reinterpret_cast<uint32_t*>(dst + 2 * lane) = pack_bf16(o_lo_x, o_lo_y);
  *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = pack_bf16(o_hi_x, o_hi_y);
}

// Backward: given dq_out/dk_out, the pre-norm qkv and rstd -> writes d(qkv) for the q and k
// columns (v columns are written by the attention backward) and accumulates dwq/dwk.
// Persistent grid; each block reduces its weight-gradient contribution in shared memory and
// issues one atomicAdd per column at the end.
__global__ void qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
                                       const __nv_bfloat16* __restrict__ qkv, long long ld, int Hq, int Hk,
                                       const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                                       const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                       const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dqkv,
                                       long long ldd, float* __restrict__ dwq, float* __restrict__ dwk, long long T,
                                       int use_norm) {
  constexpr int D = 128;
  __shared__ float sdw[2][D];
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&sdw[0][0])[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int heads = Hq + Hk;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  float accq[4] = {0, 0, 0, 0}, acck[4] = {0, 0, 0, 0};
  for (long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; gw < T * heads;
       gw += nwarps) {
    const long long t = gw / heads;
    const int h = static_cast<int>(gw - t * heads);
    const bool is_q = h < Hq;
    const __nv_bfloat16* g = is_q ? dq + (t * Hq + h) * D : dk + (t * Hk + (h - Hq)) * D;
    float2 glo = unpack_bf16(*reinterpret_cast<const uint32_t*>(g + 2 * lane));
    float2 ghi = unpack_bf16(*reinterpret_cast<const uint32_t*>(g + 64 + 2 * lane));
    const float2 c = *reinterpret_cast<const float2*>(cos_t + t * (D / 2) + 2 * lane);
    const float2 s = *reinterpret_cast<const float2*>(sin_t + t * (D / 2) + 2 * lane);
    // inverse rotation (transpose of the forward map)
    float dl_x = glo.x * c.x + ghi.x * s.x, dl_y = glo.y * c.y + ghi.y * s.y;
    float dh_x = ghi.x * c.x - glo.x * s.x, dh_y = ghi.y * c.y - glo.y * s.y;
    __nv_bfloat16* out = dqkv + t * ldd + static_cast<long long>(h) * D;
    if (use_norm) {
      const __nv_bfloat16* src = qkv + t * ld + static_cast<long long>(h) * D;
      const __nv_bfloat16* w = is_q ? wq : wk;
      float2 xlo = unpack_bf16(*reinterpret_cast<const uint32_t*>(src + 2 * lane));
      float2 xhi = unpack_bf16(*reinterpret_cast<const uint32_t*>(src + 64 + 2 * lane));
      float2 wl = unpack_bf16(*reinterpret_cast<const uint32_t*>(w + 2 * lane));
      float2 wh = unpack_bf16(*reinterpret_cast<const uint32_t*>(w + 64 + 2 * lane));
      const float rstd = rstd_in[gw];
      float xh[4] = {xlo.x * rstd, xlo.y * rstd, xhi.x * rstd, xhi.y * rstd};
      float dyv[4] = {dl_x, dl_y, dh_x, dh_y};
      float wv[4] = {wl.x, wl.y, wh.x, wh.y};
      float gg[4];
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        gg[j] = dyv[j] * wv[j];
        dot += gg[j] * xh[j];
        if (is_q) accq[j] += dyv[j] * xh[j]; else acck[j] += dyv[j] * xh[j];
      }
      dot = warp_sum(dot) / D;
      dl_x = rstd * (gg[0] - xh[0] * dot); dl_y = rstd * (gg[1] - xh[1] * dot);
      dh_x = rstd * (gg[2] - xh[2] * dot); dh_y = rstd * (gg[3] - xh[3] * dot);
    }
    *reinterpret_cast<uint32_t*>(out + 2 * lane) = pack_bf16(dl_x, dl_y);
    *reinterpret_cast<uint32_t*>(out + 64 + 2 * lane) = pack_bf16(dh_x, dh_y);
  }
  if (use_norm) {
    atomicAdd(&sdw[0][2 * lane], accq[0]); atomicAdd(&sdw[0][2 * lane + 1], accq[1]);
    atomicAdd(&sdw[0][64 + 2 * lane], accq[2]); atomicAdd(&sdw[0][64 + 2 * lane + 1], accq[3]);
    atomicAdd(&sdw[1][2 * lane], acck[0]); atomicAdd(&sdw[1][2 * lane + 1], acck[1]);
    atomicAdd(&sdw[1][64 + 2 * lane], acck[2]); atomicAdd(&sdw[1][64 + 2 * lane + 1], acck[3]);
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      atomicAdd(dwq + i, sdw[0][i]);
      atomicAdd(dwk + i, sdw[1][i]);
    }
  }
}

// ============================================================================
// SwiGLU (standalone).  x: [R, 2F] = [gate | up]; y: [R, F]; optional row_scale [R].
// ============================================================================
// `nrows` (optional, device): rows at or beyond *nrows are skipped (padded buffers whose fill is only known on the device)
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ y,
                                  long long ldy, const float* __restrict__ row_scale, long long R, int F,
                                  const int* __restrict__ nrows) {
  const long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  const long long total = R * F;
  if (idx >= total) return;
  const long long r = idx / F;
  if (nrows && r >= *nrows) return;
  const int c = static_cast<int>(idx - r * F);
  const float sc = row_scale ? row_scale[r] : 1.f;
  uint4 g = *reinterpret_cast<const uint4*>(x + r * ldx + c);
  uint4 u = *reinterpret_cast<const uint4*>(x + r * ldx + F + c);
  uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w}, os[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 gf = unpack_bf16(gs[j]), uf = unpack_bf16(us[j]);
    os[j] = pack_bf16(gf.x / (1.f + __expf(-gf.x)) * uf.x * sc, gf.y / (1.f + __expf(-gf.y)) * uf.y * sc);
  }
  *reinterpret_cast<uint4*>(y + r * ldy + c) = make_uint4(os[0], os[1], os[2], os[3]);
}

// Backward: one block per row (so the per-row d(scale) reduction is local).
//   a = silu(g) * u ; y = a * s
//   dg = dy * s * u * sig(g) * (1 + g * (1 - sig(g))) ; du = dy * s * silu(g) ; ds = sum(dy * a)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, long long lddy,
                                  const __nv_bfloat16* __restrict__ x, long long ldx,
                                  const float* __restrict__ row_scale, __nv_bfloat16* __restrict__ dx, long long lddx,
                                  float* __restrict__ dscale, int F, const int* __restrict__ nrows) {
  __shared__ float red[32];
  const long long r = blockIdx.x;
  if (nrows && r >= *nrows) return;
  const float sc = row_scale ? row_scale[r] : 1.f;
  float ds = 0.f;
  for (int c = threadIdx.x * 8; c < F; c += blockDim.x * 8) {
    uint4 g = *reinterpret_cast<const uint4*>(x + r * ldx + c);
    uint4 u = *reinterpret_cast<const uint4*>(x + r * ldx + F + c);
    uint4 d = *reinterpret_cast<const uint4*>(dy + r * lddy + c);
    uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w}, dsrc[4] = {d.x, d.y, d.z, d.w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 gf = unpack_bf16(gs[j]), uf = unpack_bf16(us[j]), df = unpack_bf16(dsrc[j]);
      float sg0 = 1.f / (1.f + __expf(-gf.x)), sg1 = 1.f / (1.f + __expf(-gf.y));
      float si0 = gf.x * sg0, si1 = gf.y * sg1;
      ds += df.x * si0 * uf.x + df.y * si1 * uf.y;
      float d0 = df.x * sc, d1 = df.y * sc;
      og[j] = pack_bf16(d0 * uf.x * sg0 * (1.f + gf.x * (1.f - sg0)), d1 * uf.y * sg1 * (1.f + gf.y * (1.f - sg1)));
      ou[j] = pack_bf16(d0 * si0, d1 * si1);
    }
    *reinterpret_cast<uint4*>(dx + r * lddx + c) = make_uint4(og[0], og[1], og[2], og[3]);
    *reinterpret_cast<uint4*>(dx + r * lddx + F + c) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
  if (dscale) {
    ds = block_sum(ds, red);
    if (threadIdx.x == 0) dscale[r] = ds;
  }
}

// ============================================================================
// Cross-entropy over logits [R, V] (bf16 or fp32), labels int64, ignore_index < 0.
// Writes per-row loss (0 for ignored rows) and, when dlogits != nullptr, the gradient
// (softmax - onehot) * grad_scale[0] in bf16 (may alias a bf16 logits buffer).
// ============================================================================
template <typename TL>
__device__ __forceinline__ float ld_logit(const TL* p, long long i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

template <typename TL>
__global__ void __launch_bounds__(1024)
cross_entropy_kernel(const TL* __restrict__ logits, long long ldl, const long long* __restrict__ labels,
                     float* __restrict__ loss_rows, float* __restrict__ lse_rows, __nv_bfloat16* dlogits, long long ldd,
                     const float* __restrict__ grad_scale, float grad_scale_host, int V) {
  __shared__ float red[32];
  const long long r = blockIdx.x;
  const TL* lr = logits + r * ldl;
  const long long label = labels[r];
  const bool valid = label >= 0 && label < V;
  constexpr bool kBf16 = sizeof(TL) == 2;
  // 16-byte vector path for bf16 rows (8 logits per access); everything else goes element by element
  const bool vec = kBf16 && (V % 8 == 0) && ((reinterpret_cast<uintptr_t>(lr) & 15) == 0) &&
                   (dlogits == nullptr || (reinterpret_cast<uintptr_t>(dlogits + r * ldd) & 15) == 0);
  if (!valid) {
    if (threadIdx.x == 0) { loss_rows[r] = 0.f; if (lse_rows) lse_rows[r] = 0.f; }
    if (dlogits) {
      if (vec) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) *reinterpret_cast<uint4*>(dlogits + r * ldd + c) = z;
      } else {
        __nv_bfloat16 z = __float2bfloat16(0.f);
        for (int c = threadIdx.x; c < V; c += blockDim.x) dlogits[r * ldd + c] = z;
      }
    }
    return;
  }
  float m = -INFINITY, s = 0.f;
  if (vec) {
    const __nv_bfloat16* lb = reinterpret_cast<const __nv_bfloat16*>(lr);
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(lb + c);
      const float2 a = unpack_bf16(u.x), b2 = unpack_bf16(u.y), c2 = unpack_bf16(u.z), d = unpack_bf16(u.w);
      const float f[8] = {a.x, a.y, b2.x, b2.y, c2.x, c2.y, d.x, d.y};
      float vm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) vm = fmaxf(vm, f[j]);
      if (vm > m) { s *= __expf(m - vm); m = vm; }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
    }
  } else {
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
      float v = ld_logit<TL>(lr, c);
      if (v > m) { s = s * __expf(m - v) + 1.f; m = v; } else { s += __expf(v - m); }
    }
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(s, red);
  const float lse = gm + logf(gs);
  if (threadIdx.x == 0) {
    loss_rows[r] = lse - ld_logit<TL>(lr, label);
    if (lse_rows) lse_rows[r] = lse;
  }
  if (dlogits) {
    const float sc = (grad_scale ? grad_scale[0] : 1.f) * grad_scale_host;
    __syncthreads();  // the label logit has been read before any thread overwrites an aliased buffer
    if (vec) {
      const __nv_bfloat16* lb = reinterpret_cast<const __nv_bfloat16*>(lr);
      for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
        const uint4 u = *reinterpret_cast<const uint4*>(lb + c);
        const float2 a = unpack_bf16(u.x), b2 = unpack_bf16(u.y), c2 = unpack_bf16(u.z), d = unpack_bf16(u.w);
        float f[8] = {a.x, a.y, b2.x, b2.y, c2.x, c2.y, d.x, d.y};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float pr = __expf(f[j] - lse);
          if (c + j == label) pr -= 1.f;
          f[j] = pr * sc;
        }
        uint4 o;
        o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]); o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
        *reinterpret_cast<uint4*>(dlogits + r * ldd + c) = o;
      }
    } else {
      for (int c = threadIdx.x; c < V; c += blockDim.x) {
        float pr = __expf(ld_logit<TL>(lr, c) - lse);
        if (c == label) pr -= 1.f;
        dlogits[r * ldd + c] = __float2bfloat16(pr * sc);
      }
    }
  }
}

// ============================================================================
// Multi-tensor AdamW on fp32 master shards with optional bf16 shadow copy.
// meta[i] = {p, g, m, v, shadow_bf16 (or 0), numel, g_is_bf16}; chunk table maps
// blockIdx.x -> (tensor, first element).  clip_coef (device scalar, may be null)
// multiplies every gradient; the update is skipped if it is not finite.
// ============================================================================
struct AdamMeta {
  float* p;
  const void* g;
  float* m;
  float* v;
  __nv_bfloat16* shadow;
  long long numel;
  long long g_is_bf16;
};
constexpr int ADAM_CHUNK = 65536;

__device__ __forceinline__ void adamw_one(float& p, float g, float& m, float& v, float lr, float beta1, float beta2,
                                          float eps, float decay, float step_size, float bc2_sqrt) {
  p *= decay;
  m = m + (1.f - beta1) * (g - m);
  v = beta2 * v + (1.f - beta2) * g * g;
  p -= step_size * m / (sqrtf(v) / bc2_sqrt + eps);
}

__global__ void __launch_bounds__(256)
adamw_kernel(const AdamMeta* __restrict__ meta, const int2* __restrict__ chunks, float lr, float beta1, float beta2,
             float eps, float weight_decay, float bc1, float bc2_sqrt, const float* __restrict__ clip_coef,
             float grad_prescale) {
  const int2 ch = chunks[blockIdx.x];
  const AdamMeta t = meta[ch.x];
  const long long start = static_cast<long long>(ch.y) * ADAM_CHUNK;
  long long end = start + ADAM_CHUNK;
  if (end > t.numel) end = t.numel;
  float coef = grad_prescale;
  if (clip_coef) {
    float c = clip_coef[0];
    if (!isfinite(c)) return;
    coef *= c;
  }
  const float step_size = lr / bc1;
  const float decay = 1.f - lr * weight_decay;
  const bool aligned = ((reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.m) |
                         reinterpret_cast<uintptr_t>(t.v) | reinterpret_cast<uintptr_t>(t.g) |
                         reinterpret_cast<uintptr_t>(t.shadow)) & 15) == 0;
  const long long n4 = aligned ? ((end - start) / 4) : 0;
  for (long long q = threadIdx.x; q < n4; q += blockDim.x) {
    const long long i = start + q * 4;
    float4 p = *reinterpret_cast<const float4*>(t.p + i);
    float4 m = *reinterpret_cast<const float4*>(t.m + i);
    float4 v = *reinterpret_cast<const float4*>(t.v + i);
    float g[4];
    if (t.g_is_bf16) {
      const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(t.g) + i);
      const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    } else {
      const float4 u = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(t.g) + i);
      g[0] = u.x; g[1] = u.y; g[2] = u.z; g[3] = u.w;
    }
    adamw_one(p.x, g[0] * coef, m.x, v.x, lr, beta1, beta2, eps, decay, step_size, bc2_sqrt);
    adamw_one(p.y, g[1] * coef, m.y, v.y, lr, beta1, beta2, eps, decay, step_size, bc2_sqrt);
    adamw_one(p.z, g[2] * coef, m.z, v.z, lr, beta1, beta2, eps, decay, step_size, bc2_sqrt);
    adamw_one(p.w, g[3] * coef, m.w, v.w, lr, beta1, beta2, eps, decay, step_size, bc2_sqrt);
    *reinterpret_cast<float4*>(t.p + i) = p;
    *reinterpret_cast<float4*>(t.m + i) = m;
    *reinterpret_cast<float4*>(t.v + i) = v;
    if (t.shadow) {
      uint2 o;
      o.x = pack_bf16(p.x, p.y); o.y = pack_bf16(p.z, p.w);
      *reinterpret_cast<uint2*>(t.shadow + i) = o;
    }
  }
  for (long long i = start + n4 * 4 + threadIdx.x; i < end; i += blockDim.x) {
    float g = t.g_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(t.g)[i])
                          : reinterpret_cast<const float*>(t.g)[i];
    float p = t.p[i], m = t.m[i], v = t.v[i];
    adamw_one(p, g * coef, m, v, lr, beta1, beta2, eps, decay, step_size, bc2_sqrt);
    t.p[i] = p; t.m[i] = m; t.v[i] = v;
    if (t.shadow) t.shadow[i] = __float2bfloat16(p);
  }
}

// Squared-norm partials: partial[blockIdx.x] = sum over the chunk of g^2 (fp32).
__global__ void __launch_bounds__(256)
sqnorm_kernel(const AdamMeta* __restrict__ meta, const int2* __restrict__ chunks, float* __restrict__ partial,
              float prescale) {
  __shared__ float red[32];
  const int2 ch = chunks[blockIdx.x];
  const AdamMeta t = meta[ch.x];
  const long long start = static_cast<long long>(ch.y) * ADAM_CHUNK;
  long long end = start + ADAM_CHUNK;
  if (end > t.numel) end = t.numel;
  float s = 0.f;
  const bool aligned = (reinterpret_cast<uintptr_t>(t.g) & 15) == 0;
  const long long n8 = (aligned && t.g_is_bf16) ? ((end - start) / 8) : 0;
  for (long long q = threadIdx.x; q < n8; q += blockDim.x) {
    const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(t.g) + start + q * 8);
    const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
    s += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
  }
  for (long long i = start + n8 * 8 + threadIdx.x; i < end; i += blockDim.x) {
    float g = t.g_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(t.g)[i])
                          : reinterpret_cast<const float*>(t.g)[i];
    s += g * g;
  }
  s = block_sum(s, red) * prescale * prescale;
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// out[0] = sum(partial[0..n)) + extra_sq ; out[1] = sqrt(out[0]) ; out[2] = min(1, max_norm/(norm+1e-6))
__global__ void clip_coef_kernel(const float* __restrict__ partial, int n, const float* __restrict__ extra_sq,
                                 float max_norm, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    if (extra_sq) s += extra_sq[0];
    float norm = sqrtf(s);
    out[0] = s;
    out[1] = norm;
    float c = max_norm / (norm + 1e-6f);
    out[2] = (max_norm > 0.f) ? fminf(c, 1.f) : 1.f;
    if (!isfinite(norm)) out[2] = norm;  // propagates NaN/Inf so the update is skipped
  }
}

}  // namespace ttb

// ----------------------------------------------------------------------------
// C ABI
// ----------------------------------------------------------------------------
using namespace ttb;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_RET() do { cudaError_t e__ = cudaGetLastError(); return e__ == cudaSuccess ? 0 : 400 + (int)e__; } while (0)

TTB_EXPORT int ttb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* sum_out,
                               float* rstd, long long T, int H, float eps, int one_plus_w, void* stream) {
  if (H % 8) return 901;
  if (T == 0) return 0;
  int threads = H / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  const int iters = (H + threads * 8 - 1) / (threads * 8);
  auto X = (const __nv_bfloat16*)x; auto R = (const __nv_bfloat16*)residual; auto W = (const __nv_bfloat16*)w;
  if (iters <= 1) rmsnorm_fwd_kernel<1><<<(unsigned)T, threads, 0, STREAM(stream)>>>(X, R, W, (__nv_bfloat16*)y, (__nv_bfloat16*)sum_out, rstd, H, eps, one_plus_w);
  else if (iters <= 4) rmsnorm_fwd_kernel<4><<<(unsigned)T, threads, 0, STREAM(stream)>>>(X, R, W, (__nv_bfloat16*)y, (__nv_bfloat16*)sum_out, rstd, H, eps, one_plus_w);
  else return 902;
  LAUNCH_RET();
}

// dw_partial must hold grid*H floats; returns the grid size used through *grid_out.
TTB_EXPORT int ttb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in,
                               void* dx, float* dw_partial, float* dw_out, long long T, int H, int one_plus_w,
                               int grid, void* stream) {
  if (H % 8) return 901;
  if (T == 0) return 0;
  int threads = H / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  const int iters = (H + threads * 8 - 1) / (threads * 8);
  if (grid > T) grid = (int)T;
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  if (iters <= 1) rmsnorm_bwd_kernel<1><<<grid, threads, 0, STREAM(stream)>>>(DY, X, W, rstd, (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, dw_partial, T, H, one_plus_w);
  else if (iters <= 4) rmsnorm_bwd_kernel<4><<<grid, threads, 0, STREAM(stream)>>>(DY, X, W, rstd, (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, dw_partial, T, H, one_plus_w);
  else return 902;
  colsum_kernel<<<(H + 255) / 256, 256, 0, STREAM(stream)>>>(dw_partial, dw_out, grid, H);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                                 long long T, int H, float eps, void* stream) {
  if (H % 8) return 901;
  if (T == 0) return 0;
  int threads = H / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  const int iters = (H + threads * 8 - 1) / (threads * 8);
  auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w; auto B = (const __nv_bfloat16*)b;
  if (iters <= 1) layernorm_fwd_kernel<1><<<(unsigned)T, threads, 0, STREAM(stream)>>>(X, W, B, (__nv_bfloat16*)y, mean, rstd, H, eps);
  else if (iters <= 4) layernorm_fwd_kernel<4><<<(unsigned)T, threads, 0, STREAM(stream)>>>(X, W, B, (__nv_bfloat16*)y, mean, rstd, H, eps);
  else return 902;
  LAUNCH_RET();
}

// part must hold grid * 2 * H floats; dwdb_out receives [2][H] (dw then db).
TTB_EXPORT int ttb_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                                 float* part, float* dwdb_out, long long T, int H, int grid, void* stream) {
  if (H % 8) return 901;
  if (T == 0) return 0;
  int threads = H / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  const int iters = (H + threads * 8 - 1) / (threads * 8);
  if (grid > T) grid = (int)T;
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  if (iters <= 1) layernorm_bwd_kernel<1><<<grid, threads, 0, STREAM(stream)>>>(DY, X, W, mean, rstd, (__nv_bfloat16*)dx, part, T, H);
  else if (iters <= 4) layernorm_bwd_kernel<4><<<grid, threads, 0, STREAM(stream)>>>(DY, X, W, mean, rstd, (__nv_bfloat16*)dx, part, T, H);
  else return 902;
  colsum_kernel<<<(2 * H + 255) / 256, 256, 0, STREAM(stream)>>>(part, dwdb_out, grid, 2 * H);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_bias_act_fwd(const void* x, const void* bias, const void* residual, void* y, long long R, int C, int act,
                                void* stream) {
  if (C % 8 || act < 0 || act > 2) return 901;
  if (R == 0) return 0;
  const long long total = R * (C / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  bias_act_fwd_kernel<<<(unsigned)blocks, 256, 0, STREAM(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)bias,
                                                                    (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, R, C, act);
  LAUNCH_RET();
}

// part must hold grid * C floats; dx may be null (identity activation: d(x) is dy itself).
TTB_EXPORT int ttb_bias_act_bwd(const void* dy, const void* x, const void* bias, void* dx, float* part, float* dbias_out,
                                long long R, int C, int act, int grid, void* stream) {
  if (C % 8 || act < 0 || act > 2) return 901;
  if (R == 0) return 0;
  int threads = C / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  const int iters = (C + threads * 8 - 1) / (threads * 8);
  if (grid > R) grid = (int)R;
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto B = (const __nv_bfloat16*)bias;
  if (iters <= 1) bias_act_bwd_kernel<1><<<grid, threads, 0, STREAM(stream)>>>(DY, X, B, (__nv_bfloat16*)dx, part, R, C, act);
  else if (iters <= 4) bias_act_bwd_kernel<4><<<grid, threads, 0, STREAM(stream)>>>(DY, X, B, (__nv_bfloat16*)dx, part, R, C, act);
  else if (iters <= 8) bias_act_bwd_kernel<8><<<grid, threads, 0, STREAM(stream)>>>(DY, X, B, (__nv_bfloat16*)dx, part, R, C, act);
  else return 902;
  colsum_kernel<<<(C + 255) / 256, 256, 0, STREAM(stream)>>>(part, dbias_out, grid, C);
  LAUNCH_RET();
}

static void conv_grid(long long T, int D, int& threads, dim3& grid, int& rows_per_block) {
  const int vec = D / 8;
  threads = vec >= 128 ? 128 : ((vec + 31) / 32) * 32;
  const int gx = (vec + threads - 1) / threads;
  long long want = (148LL * 8 + gx - 1) / gx;      // about eight blocks per SM in total
  if (want > T) want = T;
  if (want < 1) want = 1;
  rows_per_block = static_cast<int>((T + want - 1) / want);
  grid = dim3(gx, static_cast<unsigned>((T + rows_per_block - 1) / rows_per_block));
}

TTB_EXPORT int ttb_causal_conv1d_fwd(const void* x, const void* w, const void* bias, const int* seq_start, void* y,
                                     long long T, int D, int W, int silu, void* stream) {
  if (D % 8 || W < 1 || W > CONV_MAX_W) return 901;
  if (T == 0) return 0;
  int threads, rpb;
  dim3 grid;
  conv_grid(T, D, threads, grid, rpb);
  if (W <= 4)
    causal_conv1d_kernel<false, 4><<<grid, threads, 0, STREAM(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
        (const __nv_bfloat16*)bias, seq_start, nullptr, (__nv_bfloat16*)y, nullptr, T, D, W, silu, rpb);
  else
    causal_conv1d_kernel<false, 8><<<grid, threads, 0, STREAM(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
        (const __nv_bfloat16*)bias, seq_start, nullptr, (__nv_bfloat16*)y, nullptr, T, D, W, silu, rpb);
  LAUNCH_RET();
}

// part must hold row_blocks * (W + 1) * D floats (row_blocks from ttb_causal_conv1d_row_blocks); dwdb_out: [(W + 1), D]
TTB_EXPORT int ttb_causal_conv1d_row_blocks(long long T, int D) {
  int threads, rpb;
  dim3 grid;
  conv_grid(T > 0 ? T : 1, D, threads, grid, rpb);
  return static_cast<int>(grid.y);
}

TTB_EXPORT int ttb_causal_conv1d_bwd(const void* dy, const void* x, const void* w, const void* bias, const int* seq_start,
                                     const int* seq_end, void* dpre, void* dx, float* part, float* dwdb_out, long long T,
                                     int D, int W, int silu, void* stream) {
  if (D % 8 || W < 1 || W > CONV_MAX_W) return 901;
  if (T == 0) return 0;
  int threads, rpb;
  dim3 grid;
  conv_grid(T, D, threads, grid, rpb);
  if (W <= 4) {
    causal_conv1d_kernel<true, 4><<<grid, threads, 0, STREAM(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
        (const __nv_bfloat16*)bias, seq_start, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dpre, part, T, D, W, silu, rpb);
    causal_conv1d_dx_kernel<4><<<grid, threads, 0, STREAM(stream)>>>((const __nv_bfloat16*)dpre, (const __nv_bfloat16*)w,
                                                                     seq_end, (__nv_bfloat16*)dx, T, D, W, rpb);
  } else {
    causal_conv1d_kernel<true, 8><<<grid, threads, 0, STREAM(stream)>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
        (const __nv_bfloat16*)bias, seq_start, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dpre, part, T, D, W, silu, rpb);
    causal_conv1d_dx_kernel<8><<<grid, threads, 0, STREAM(stream)>>>((const __nv_bfloat16*)dpre, (const __nv_bfloat16*)w,
                                                                     seq_end, (__nv_bfloat16*)dx, T, D, W, rpb);
  }
  const int cols = (W + 1) * D;
  colsum_kernel<<<(cols + 255) / 256, 256, 0, STREAM(stream)>>>(part, dwdb_out, static_cast<int>(grid.y), cols);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_qknorm_rope_fwd(const void* qkv, long long ld, int Hq, int Hk, int D, const void* wq, const void* wk,
                                   const float* cos_t, const float* sin_t, void* q_out, void* k_out, float* rstd,
                                   long long T, float eps, int use_norm, void* stream) {
  if (D != 128) return 901;
  const long long warps = T * (Hq + Hk);
  if (warps == 0) return 0;
  const long long blocks = (warps + 7) / 8;
  qknorm_rope_fwd_kernel<<<(unsigned)blocks, 256, 0, STREAM(stream)>>>(
      (const __nv_bfloat16*)qkv, ld, Hq, Hk, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, cos_t, sin_t,
      (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, rstd, T, eps, use_norm);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_qknorm_rope_bwd(const void* dq, const void* dk, const void* qkv, long long ld, int Hq, int Hk, int D,
                                   const void* wq, const void* wk, const float* cos_t, const float* sin_t,
                                   const float* rstd, void* dqkv, long long ldd, float* dwq, float* dwk, long long T,
                                   int use_norm, int grid, void* stream) {
  if (D != 128) return 901;
  if (T == 0) return 0;
  qknorm_rope_bwd_kernel<<<grid, 256, 0, STREAM(stream)>>>(
      (const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)qkv, ld, Hq, Hk,
      (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, cos_t, sin_t, rstd, (__nv_bfloat16*)dqkv, ldd, dwq, dwk, T,
      use_norm);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_swiglu_fwd(const void* x, long long ldx, void* y, long long ldy, const float* row_scale, long long R,
                              int F, const int* nrows, void* stream) {
  if (F % 8 || ldx % 8 || ldy % 8) return 901;
  const long long n = R * F / 8;
  if (n == 0) return 0;
  swiglu_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, STREAM(stream)>>>((const __nv_bfloat16*)x, ldx,
                                                                            (__nv_bfloat16*)y, ldy, row_scale, R, F, nrows);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_swiglu_bwd(const void* dy, long long lddy, const void* x, long long ldx, const float* row_scale,
                              void* dx, long long lddx, float* dscale, long long R, int F, const int* nrows, void* stream) {
  if (F % 8 || ldx % 8 || lddy % 8 || lddx % 8) return 901;
  if (R == 0) return 0;
  int threads = F / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  swiglu_bwd_kernel<<<(unsigned)R, threads, 0, STREAM(stream)>>>((const __nv_bfloat16*)dy, lddy,
                                                                (const __nv_bfloat16*)x, ldx, row_scale,
                                                                (__nv_bfloat16*)dx, lddx, dscale, F, nrows);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_cross_entropy(const void* logits, int logits_fp32, long long ldl, const long long* labels,
                                 float* loss_rows, float* lse_rows, void* dlogits, long long ldd,
                                 const float* grad_scale, float grad_scale_host, long long R, int V, void* stream) {
  if (R == 0) return 0;
  if (logits_fp32)
    cross_entropy_kernel<float><<<(unsigned)R, 1024, 0, STREAM(stream)>>>(
        (const float*)logits, ldl, labels, loss_rows, lse_rows, (__nv_bfloat16*)dlogits, ldd, grad_scale,
        grad_scale_host, V);
  else
    cross_entropy_kernel<__nv_bfloat16><<<(unsigned)R, 1024, 0, STREAM(stream)>>>(
        (const __nv_bfloat16*)logits, ldl, labels, loss_rows, lse_rows, (__nv_bfloat16*)dlogits, ldd, grad_scale,
        grad_scale_host, V);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_adam_chunk_elems() { return ADAM_CHUNK; }

TTB_EXPORT int ttb_adamw(const void* meta, const void* chunks, int n_chunks, float lr, float beta1, float beta2,
                         float eps, float weight_decay, float bc1, float bc2_sqrt, const float* clip_coef,
                         float grad_prescale, void* stream) {
  if (n_chunks == 0) return 0;
  adamw_kernel<<<n_chunks, 256, 0, STREAM(stream)>>>((const AdamMeta*)meta, (const int2*)chunks, lr, beta1, beta2, eps,
                                                     weight_decay, bc1, bc2_sqrt, clip_coef, grad_prescale);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_grad_sqnorm(const void* meta, const void* chunks, int n_chunks, float* partial, float prescale,
                               void* stream) {
  if (n_chunks == 0) return 0;
  sqnorm_kernel<<<n_chunks, 256, 0, STREAM(stream)>>>((const AdamMeta*)meta, (const int2*)chunks, partial, prescale);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_clip_coef(const float* partial, int n, const float* extra_sq, float max_norm, float* out3,
                             void* stream) {
  clip_coef_kernel<<<1, 1024, 0, STREAM(stream)>>>(partial, n, extra_sq, max_norm, out3);
  LAUNCH_RET();
}

// ----------------------------------------------------------------------------
// Allocation-free RMSNorm backward (see ttb_noalloc.h for the contract).
// The scratch that ttb_rmsnorm_bwd receives from its caller lives here in a file-scope device array.  In host code
// the name `g_noalloc_scratch` is only a handle for the runtime; the address a kernel can use comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
// ----------------------------------------------------------------------------
#include "ttb_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[TTB_NOALLOC_BLOCKS * TTB_NOALLOC_MAX_H];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (cached).  Returns 0 or a TTB_NOALLOC_ERR_SYMBOL code.
int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TTB_NOALLOC_ERR_SYMBOL + static_cast<int>(e);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) return TTB_NOALLOC_ERR_SYMBOL + static_cast<int>(e);
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

TTB_EXPORT int ttb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                       const void* dres_in, void* dx, float* dw_out, long long T, int H,
                                       int one_plus_w, void* stream) {
  if (H <= 0 || (H % 8) != 0 || H > TTB_NOALLOC_MAX_H || T < 0) return TTB_NOALLOC_ERR_SIZE;
  if (T == 0) return TTB_NOALLOC_OK;
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != 0) return rc;
  int threads = H / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  const int iters = (H + threads * 8 - 1) / (threads * 8);
  int grid = TTB_NOALLOC_BLOCKS;
  if (grid > T) grid = static_cast<int>(T);
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto W = (const __nv_bfloat16*)w;
  // every block writes its full row of `scratch` (H floats), and the column sum below reads exactly rows [0, grid):
  // nothing has to be cleared between calls
  if (iters <= 1)
    rmsnorm_bwd_kernel<1><<<grid, threads, 0, STREAM(stream)>>>(DY, X, W, rstd, (const __nv_bfloat16*)dres_in,
                                                               (__nv_bfloat16*)dx, scratch, T, H, one_plus_w);
  else
    rmsnorm_bwd_kernel<4><<<grid, threads, 0, STREAM(stream)>>>(DY, X, W, rstd, (const __nv_bfloat16*)dres_in,
                                                               (__nv_bfloat16*)dx, scratch, T, H, one_plus_w);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return TTB_NOALLOC_ERR_LAUNCH_DX + static_cast<int>(e);
  colsum_kernel<<<(H + 255) / 256, 256, 0, STREAM(stream)>>>(scratch, dw_out, grid, H);
  e = cudaGetLastError();
  return e == cudaSuccess ? TTB_NOALLOC_OK : TTB_NOALLOC_ERR_LAUNCH_DW + static_cast<int>(e);
}

TTB_EXPORT const char* ttb_noalloc_strerror(int code) {
  if (code == TTB_NOALLOC_OK) return "ok";
  if (code == TTB_NOALLOC_ERR_SIZE)
    return "ttb_rmsnorm_bwd_noalloc: H must be a positive multiple of 8 and at most 8192 (TTB_NOALLOC_MAX_H), T >= 0";
  if (code >= TTB_NOALLOC_ERR_SYMBOL && code < TTB_NOALLOC_ERR_SYMBOL + 10000)
    return "ttb_rmsnorm_bwd_noalloc: could not resolve the device address of the built-in scratch array "
           "(cudaGetDevice / cudaGetSymbolAddress failed; code - 200000 is the CUDA error)";
  if (code >= TTB_NOALLOC_ERR_LAUNCH_DW && code < TTB_NOALLOC_ERR_LAUNCH_DW + 10000)
    return "ttb_rmsnorm_bwd_noalloc: launch of the weight-gradient column sum failed (code - 110000 is the CUDA error)";
  if (code >= TTB_NOALLOC_ERR_LAUNCH_DX && code < TTB_NOALLOC_ERR_LAUNCH_DX + 10000)
    return "ttb_rmsnorm_bwd_noalloc: launch of the dx / partial-sum kernel failed (code - 100000 is the CUDA error)";
  return "ttb_rmsnorm_bwd_noalloc: unknown error code";
}
