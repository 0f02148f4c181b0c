// In-kernel NVLink communication for expert parallelism (and other all-to-all shaped exchanges).
//
// Every rank owns one symmetric buffer (peer-mapped through CUDA IPC / VMM by the host runtime) and holds a
// table with the base address of every peer's buffer.  Kernels here move data with plain peer stores / loads
// (no NCCL, no multicast loads) and synchronise with per-(kind, source rank) epoch flags:
//   writer : data stores -> __threadfence_system() -> st.release.sys flag = epoch
//   reader : ld.acquire.sys flag until it equals epoch (bounded by a time budget) -> data loads
// A wait that exceeds its budget records {kernel, site, peer} in the status word and returns; the kernel then
// stops touching remote memory and exits, so a missing peer can never hang the GPU.
//
//   ep_exchange : per-expert token counts -> every peer; then each rank derives, from the full [W, E] matrix,
//                 (a) for its own experts: 128-row aligned segment starts, tile->expert map, rows per expert,
//                 (b) for every global expert: the first row *this* rank may write on the owning rank.
//   ep_scatter  : token rows (and routing probabilities) written straight into the owner's expert-major buffer.
//   ep_gather   : k-way sum of expert output rows pulled from the owners (+ residual), token order.
//   flag_signal / flag_wait : stream-ordered hand-offs between the kernels above and the grouped GEMMs.
//
// Together they replace counts all-gather + host read of split sizes + two all-to-all-v + chunk sort + unpermute of
// the reference dispatcher (models/modules/moe/token_dispatcher.py:125-259).
#include "peer.cuh"

namespace ttb {

constexpr int EP_ALIGN = 128;

// ------------------------------------------------------------------------------------------------------------
// counts exchange + layout tables.  One CTA.
//   symmetric layout (per rank): counts_all int32 [W][E] at byte offset off_counts; flags int32 [W] at off_flags
// ------------------------------------------------------------------------------------------------------------
struct EpExchangeParams {
  PeerTable peers;
  long long off_counts, off_flags;
  const int* counts;   // [E] local routing counts
  int rank, W, E, epoch;
  unsigned long long budget_ns;
  int m_tiles_cap;
  int* seg_start;      // [El + 1]
  int* recv_counts;    // [El]
  int* tile_group;     // [m_tiles_cap]
  int* dest_base;      // [E]
  int* status;         // [1] 0 ok, else error code (timeout or capacity overflow)
  int* send_base;      // [E] optional: first position of every expert's rows in this rank's send order
};

__global__ void ep_exchange_kernel(const EpExchangeParams p) {
  extern __shared__ int sh[];  // [W*E] counts matrix, then [W * (El+1)] per-owner segment starts
  const int W = p.W, E = p.E, El = E / W;
  int* s_counts = sh;
  int* s_seg = sh + W * E;  // s_seg[o * (El + 1) + e_l]
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  // 1. publish my counts to every peer
  for (int i = threadIdx.x; i < W * E; i += blockDim.x) {
    const int peer = i / E, e = i - peer * E;
    int* dst = reinterpret_cast<int*>(p.peers.base[peer] + p.off_counts) + p.rank * E + e;
    *dst = p.counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < W) {
    int* f = reinterpret_cast<int*>(p.peers.base[threadIdx.x] + p.off_flags) + p.rank;
    st_release_sys(f, p.epoch);
  }
  // 2. wait for every peer's counts (a workspace that has already failed does not wait: its peers have their answer
  //    above, and this layer's exchange is dropped like the rest of the step)
  if (threadIdx.x < W) {
    const int* f = reinterpret_cast<const int*>(p.peers.base[p.rank] + p.off_flags) + threadIdx.x;
    if (*reinterpret_cast<volatile int*>(p.status) != 0 || !wait_flag(f, p.epoch, p.budget_ns, 1, threadIdx.x, p.status))
      s_ok = 0;
  }
  __syncthreads();
  // a peer never answered, or (below) some owner's receive buffer is too small for this batch: leave tables that make
  // every later kernel of this layer a no-op (no rows, no tiles, destination rows outside the buffer, which the
  // senders skip) instead of uninitialised indices or rows past the end of a buffer
  auto no_op_tables = [&]() {
    for (int e = threadIdx.x; e < E; e += blockDim.x) p.dest_base[e] = -(1 << 30);
    for (int el = threadIdx.x; el <= El; el += blockDim.x) {
      p.seg_start[el] = 0;
      if (el < El) p.recv_counts[el] = 0;
    }
    for (int m = threadIdx.x; m < p.m_tiles_cap; m += blockDim.x) p.tile_group[m] = -1;
    if (p.send_base)
      for (int e = threadIdx.x; e < E; e += blockDim.x) p.send_base[e] = 0;
  };
  if (!s_ok) {
    no_op_tables();
    return;
  }
  const int* mine = reinterpret_cast<const int*>(p.peers.base[p.rank] + p.off_counts);
  for (int i = threadIdx.x; i < W * E; i += blockDim.x) s_counts[i] = mine[i];
  __syncthreads();
  // 3. per-owner aligned segment starts (thread o scans owner o's local experts)
  if (threadIdx.x < W) {
    const int o = threadIdx.x;
    int acc = 0;
    for (int el = 0; el < El; ++el) {
      s_seg[o * (El + 1) + el] = acc;
      int tot = 0;
      for (int s = 0; s < W; ++s) tot += s_counts[s * E + o * El + el];
      acc += ((tot + EP_ALIGN - 1) / EP_ALIGN) * EP_ALIGN;
    }
    s_seg[o * (El + 1) + El] = acc;
    // receive capacity exceeded on owner `o` (every rank sees the whole matrix, so all of them drop this layer's
    // exchange together; the status makes the step fail before the optimizer runs)
    if (acc > p.m_tiles_cap * EP_ALIGN) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 2);
    no_op_tables();
    return;
  }
  // 4. tables
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int o = e / El, el = e - o * El;
    int before = 0;
    for (int s = 0; s < p.rank; ++s) before += s_counts[s * E + e];
    p.dest_base[e] = s_seg[o * (El + 1) + el] + before;
  }
  // send order of the fused dispatch: local expert index major, owners rotated from rank + 1 (own rows last), so
  // that all owners' first experts complete first and every owner receives from one source at a time
  if (p.send_base && threadIdx.x == 0) {
    int acc = 0;
    for (int el = 0; el < El; ++el)
      for (int j = 0; j < W; ++j) {
        const int e = ((p.rank + 1 + j) % W) * El + el;
        p.send_base[e] = acc;
        acc += p.counts[e];
      }
  }
  const int* my_seg = s_seg + p.rank * (El + 1);
  for (int el = threadIdx.x; el <= El; el += blockDim.x) {
    p.seg_start[el] = my_seg[el];
    if (el < El) {
      int tot = 0;
      for (int s = 0; s < W; ++s) tot += s_counts[s * E + p.rank * El + el];
      p.recv_counts[el] = tot;
    }
  }
  for (int m = threadIdx.x; m < p.m_tiles_cap; m += blockDim.x) {
    const int row = m * EP_ALIGN;
    int g = -1;
    if (row < my_seg[El]) {
      int lo = 0, hi = El;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (my_seg[mid] <= row) lo = mid; else hi = mid;
      }
      g = lo;
    }
    p.tile_group[m] = g;
  }
}

// ------------------------------------------------------------------------------------------------------------
// scatter: dst_rank = expert / El, dst_row = dest_row[n].  One warp per (token, slot) entry.
// The last block to finish publishes flag[kind][rank] = epoch on every peer.
// ------------------------------------------------------------------------------------------------------------
struct EpScatterParams {
  PeerTable peers;
  long long off_rows, off_vals, off_flags;  // byte offsets inside the symmetric buffer
  const __nv_bfloat16* src;  // [T, lds]
  long long lds;
  const int* expert;         // [N] global expert id
  const int* dest_row;       // [N]
  const float* val;          // [N] or null
  long long N;
  int k, H, El, rank, W, epoch;
  long long cap_rows;
  unsigned int* done_counter;  // local, zeroed by the launcher
  int* status;
};

__global__ void ep_scatter_kernel(const EpScatterParams p) {
  const int lane = threadIdx.x & 31;
  const long long warps_per_grid = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long n = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; n < p.N; n += warps_per_grid) {
    const int e = p.expert[n];
    const int o = e / p.El;
    const long long r = p.dest_row[n];
    if (r < 0 || r >= p.cap_rows || o < 0 || o >= p.W) {  // never write outside the peer's buffer
      if (lane == 0) atomicExch(p.status, 3);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(p.src + (n / p.k) * p.lds);
    uint4* d = reinterpret_cast<uint4*>(p.peers.base[o] + p.off_rows) + r * (p.H / 8);
    for (int c = lane; c < p.H / 8; c += 32) d[c] = s[c];
    if (p.val && lane == 0) reinterpret_cast<float*>(p.peers.base[o] + p.off_vals)[r] = p.val[n];
  }
  __threadfence_system();
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) last = (atomicAdd(p.done_counter, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last) {
    __threadfence_system();
    if (threadIdx.x < p.W) {
      int* f = reinterpret_cast<int*>(p.peers.base[threadIdx.x] + p.off_flags) + p.rank;
      st_release_sys(f, p.epoch);
    }
    if (threadIdx.x == 0) *p.done_counter = 0;
  }
}

// flag[kind][rank] = epoch on every peer (stream-ordered "my buffer is ready" hand-off)
__global__ void flag_signal_kernel(PeerTable peers, long long off_flags, int rank, int W, int epoch) {
  __threadfence_system();
  if (threadIdx.x < W) st_release_sys(reinterpret_cast<int*>(peers.base[threadIdx.x] + off_flags) + rank, epoch);
}

// wait until my flag[kind][s] == epoch for every s
__global__ void flag_wait_kernel(PeerTable peers, long long off_flags, int rank, int W, int epoch,
                                 unsigned long long budget_ns, int* status) {
  if (threadIdx.x < W)
    wait_flag(reinterpret_cast<const int*>(peers.base[rank] + off_flags) + threadIdx.x, epoch, budget_ns, 2, threadIdx.x,
              status);
}

// ------------------------------------------------------------------------------------------------------------
// gather: out[t] = sum_j w[t,j] * rows_of(owner(n))[dest_row[n]]  (+ residual[t]).  One block per token.
// ------------------------------------------------------------------------------------------------------------
struct EpGatherParams {
  PeerTable peers;
  long long off_rows;
  const int* expert;    // [T*k]
  const int* dest_row;  // [T*k]
  const float* w;       // [T*k] or null
  const __nv_bfloat16* residual;
  long long ldr;
  __nv_bfloat16* out;
  long long ldo;
  int k, H, El, W;
  long long cap_rows;
  const int* status;    // skip remote reads when a wait already failed
};

__global__ void ep_gather_kernel(const EpGatherParams p) {
  const long long t = blockIdx.x;
  const bool healthy = (p.status == nullptr) || (*p.status == 0);
  for (int c = threadIdx.x * 8; c < p.H; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (healthy) {
      for (int j = 0; j < p.k; ++j) {
        const long long n = t * p.k + j;
        const int o = p.expert[n] / p.El;
        const long long r = p.dest_row[n];
        if (r < 0 || r >= p.cap_rows || o < 0 || o >= p.W) continue;
        const float wt = p.w ? p.w[n] : 1.f;
        const uint4 u = *reinterpret_cast<const uint4*>(
            reinterpret_cast<const __nv_bfloat16*>(p.peers.base[o] + p.off_rows) + r * p.H + c);
        float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
        acc[0] += wt * a.x; acc[1] += wt * a.y; acc[2] += wt * b.x; acc[3] += wt * b.y;
        acc[4] += wt * cc.x; acc[5] += wt * cc.y; acc[6] += wt * d.x; acc[7] += wt * d.y;
      }
    }
    if (p.residual) {
      const uint4 u = *reinterpret_cast<const uint4*>(p.residual + t * p.ldr + c);
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o4;
    o4.x = pack_bf16(acc[0], acc[1]); o4.y = pack_bf16(acc[2], acc[3]);
    o4.z = pack_bf16(acc[4], acc[5]); o4.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(p.out + t * p.ldo + c) = o4;
  }
}

}  // namespace ttb

using namespace ttb;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define LAUNCH_RET() do { cudaError_t e__ = cudaGetLastError(); return e__ == cudaSuccess ? 0 : 400 + (int)e__; } while (0)

static PeerTable make_peers(const unsigned long long* ptrs, int W) {
  PeerTable t;
  for (int i = 0; i < MAX_RANKS; ++i) t.base[i] = i < W ? ptrs[i] : 0ull;
  return t;
}

TTB_EXPORT int ttb_ep_exchange(const unsigned long long* peer_ptrs, long long off_counts, long long off_flags,
                               const int* counts, int rank, int W, int E, int epoch, long long budget_ms,
                               int m_tiles_cap, int* seg_start, int* recv_counts, int* tile_group, int* dest_base,
                               int* status, void* stream) {
  if (W > MAX_RANKS || E % W || W < 1) return 901;
  const int El = E / W;
  const size_t sh = static_cast<size_t>(W) * E * 4 + static_cast<size_t>(W) * (El + 1) * 4;
  if (sh > 48 * 1024) return 902;
  EpExchangeParams p{make_peers(peer_ptrs, W), off_counts, off_flags, counts, rank, W, E, epoch,
                     static_cast<unsigned long long>(budget_ms) * 1000000ull, m_tiles_cap, seg_start, recv_counts,
                     tile_group, dest_base, status, nullptr};
  ep_exchange_kernel<<<1, 256, sh, STREAM(stream)>>>(p);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_ep_scatter(const unsigned long long* peer_ptrs, long long off_rows, long long off_vals,
                              long long off_flags, const void* src, long long lds, const int* expert,
                              const int* dest_row, const float* val, long long N, int k, int H, int El, int rank,
                              int W, int epoch, long long cap_rows, unsigned int* done_counter, int* status, int grid,
                              void* stream) {
  if (W > MAX_RANKS || H % 8 || lds % 8) return 901;
  EpScatterParams p{make_peers(peer_ptrs, W), off_rows, off_vals, off_flags, (const __nv_bfloat16*)src, lds, expert,
                    dest_row, val, N, k, H, El, rank, W, epoch, cap_rows, done_counter, status};
  if (grid < 1) grid = 1;
  ep_scatter_kernel<<<grid, 256, 0, STREAM(stream)>>>(p);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_flag_signal(const unsigned long long* peer_ptrs, long long off_flags, int rank, int W, int epoch,
                               void* stream) {
  if (W > MAX_RANKS) return 901;
  flag_signal_kernel<<<1, 32, 0, STREAM(stream)>>>(make_peers(peer_ptrs, W), off_flags, rank, W, epoch);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_flag_wait(const unsigned long long* peer_ptrs, long long off_flags, int rank, int W, int epoch,
                             long long budget_ms, int* status, void* stream) {
  if (W > MAX_RANKS) return 901;
  flag_wait_kernel<<<1, 32, 0, STREAM(stream)>>>(make_peers(peer_ptrs, W), off_flags, rank, W, epoch,
                                                 static_cast<unsigned long long>(budget_ms) * 1000000ull, status);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_ep_gather(const unsigned long long* peer_ptrs, long long off_rows, const int* expert,
                             const int* dest_row, const float* w, const void* residual, long long ldr, void* out,
                             long long ldo, long long T, int k, int H, int El, int W, long long cap_rows,
                             const int* status, void* stream) {
  if (W > MAX_RANKS || H % 8 || ldo % 8) return 901;
  if (T == 0) return 0;
  EpGatherParams p{make_peers(peer_ptrs, W), off_rows, expert, dest_row, w, (const __nv_bfloat16*)residual, ldr,
                   (__nv_bfloat16*)out, ldo, k, H, El, W, cap_rows, status};
  int threads = H / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  ep_gather_kernel<<<(unsigned)T, threads, 0, STREAM(stream)>>>(p);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_comm_status(unsigned int* out4, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out4, ttb::g_status_word, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) return (int)e;
  if (reset) {
    unsigned int z[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbol(ttb::g_status_word, z, sizeof(z));
  }
  return (int)e;
}

namespace ttb {
// out[n] = vals_of(owner(n))[dest_row[n]] : scalar pull used for the routing-probability gradient
__global__ void ep_gather_vals_kernel(PeerTable peers, long long off_vals, const int* __restrict__ expert,
                                      const int* __restrict__ dest_row, float* __restrict__ out, long long N, int El,
                                      int W, long long cap_rows, const int* status) {
  const long long n = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float v = 0.f;
  if (status == nullptr || *status == 0) {
    const int o = expert[n] / El;
    const long long r = dest_row[n];
    if (r >= 0 && r < cap_rows && o >= 0 && o < W) v = reinterpret_cast<const float*>(peers.base[o] + off_vals)[r];
  }
  out[n] = v;
}
}  // namespace ttb

TTB_EXPORT int ttb_ep_gather_vals(const unsigned long long* peer_ptrs, long long off_vals, const int* expert,
                                  const int* dest_row, float* out, long long N, int El, int W, long long cap_rows,
                                  const int* status, void* stream) {
  if (W > MAX_RANKS) return 901;
  if (N == 0) return 0;
  ttb::ep_gather_vals_kernel<<<(unsigned)((N + 255) / 256), 256, 0, STREAM(stream)>>>(make_peers(peer_ptrs, W), off_vals,
                                                                                     expert, dest_row, out, N, El, W,
                                                                                     cap_rows, status);
  LAUNCH_RET();
}

// ============================================================================================================
// Ulysses sequence parallelism over peer memory.
//
// Layouts (bf16, D = 128): a rank holds `Tl` consecutive tokens of the row and all heads; around attention it
// needs all `T = W * Tl` tokens of `Hl = H / W` heads.  Head h of local token t therefore belongs to rank
// `h / Hl`, which stores it at row `rank * Tl + t`, head `h % Hl` of its `[T, Hl, D]` buffer.
// Key / value heads are repeated `rep` times first when there are fewer of them than ranks (repeated head
// `hk * rep + i`), so a source head may have `rep` destinations; the reverse direction sums the `rep` copies.
//
//   ulysses_qkv_scatter : per-head RMSNorm + rotary embedding of q and k (the epilogue of the QKV projection)
//                         computed in registers and stored straight into the owning ranks' buffers; v heads are
//                         copied the same way.  The last block publishes "rows landed" flags.
//   ulysses_scatter     : plain seq -> head push of a `[Tl, H, D]` tensor (gradient of the attention output).
//   ulysses_gather      : head -> seq pull: `[Tl, H, D]` assembled from the owners' `[T, Hl, D]` buffers, summing
//                         replicas (attention output forward; dq / dk / dv backward).
// Replaces the three + one `all_to_all_single` calls and their pack / unpack copies
// (models/modules/attention/ulysses/ulysses.py:307-327,381-383 of the reference).
// ============================================================================================================
namespace ttb {
struct UlyQkvParams {
  PeerTable peers;
  long long off_q, off_k, off_v, off_flags;
  const __nv_bfloat16* qkv;   // [Tl, ld]: q heads, then k heads, then v heads
  long long ld;
  const __nv_bfloat16 *wq, *wk;
  const float *cos_t, *sin_t; // [Tl, 64]
  float* rstd_out;            // [Tl * (Hq + Hk)] or null
  long long Tl;
  int Hq, Hk, rep, W, rank, epoch, use_norm;
  float eps;
  unsigned int* done_counter;
};

__global__ void ulysses_qkv_scatter_kernel(const UlyQkvParams p) {
  // One warp per (token, head).  Lane l owns the four consecutive columns [4l, 4l+4): lanes 0-15 hold the first half of
  // the head, lanes 16-31 the second, so the rotary partner of a column sits in lane l ^ 16 and one 8-byte access per
  // lane moves the whole 256-byte head row.
  constexpr int D = 128;
  const int lane = threadIdx.x & 31;
  const int heads = p.Hq + 2 * p.Hk;
  const int Hql = p.Hq / p.W, Hkl = p.Hk * p.rep / p.W;
  const long long total = p.Tl * heads;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const bool low = lane < 16;
  const int pair = (lane & 15) * 4;                    // rotary pair index of this lane's first column
  for (long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; gw < total; gw += nwarps) {
    const long long t = gw / heads;
    const int h = static_cast<int>(gw - t * heads);
    const __nv_bfloat16* src = p.qkv + t * p.ld + static_cast<long long>(h) * D;
    uint2 raw = *reinterpret_cast<const uint2*>(src + 4 * lane);
    const bool is_q = h < p.Hq, is_k = !is_q && h < p.Hq + p.Hk;
    if (is_q || is_k) {
      float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y);
      float x[4] = {a.x, a.y, b.x, b.y};
      float rstd = 1.f;
      if (p.use_norm) {
        const __nv_bfloat16* w = is_q ? p.wq : p.wk;
        const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
        rstd = rsqrtf(ss / D + p.eps);
        const uint2 wr = *reinterpret_cast<const uint2*>(w + 4 * lane);
        const float2 w0 = unpack_bf16(wr.x), w1 = unpack_bf16(wr.y);
        const float wv[4] = {w0.x, w0.y, w1.x, w1.y};
#pragma unroll
        for (int i = 0; i < 4; ++i)
          x[i] = __bfloat162float(__float2bfloat16(__bfloat162float(__float2bfloat16(x[i] * rstd)) * wv[i]));
      }
      if (p.rstd_out && lane == 0) p.rstd_out[t * (p.Hq + p.Hk) + h] = rstd;
      const float4 c = *reinterpret_cast<const float4*>(p.cos_t + t * (D / 2) + pair);
      const float4 s4 = *reinterpret_cast<const float4*>(p.sin_t + t * (D / 2) + pair);
      const float cv[4] = {c.x, c.y, c.z, c.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
      float o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
        // first half: x1 * cos - x2 * sin ; second half: x2 * cos + x1 * sin
        o[i] = low ? (x[i] * cv[i] - other * sv[i]) : (x[i] * cv[i] + other * sv[i]);
      }
      raw = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
    }
    const long long row = static_cast<long long>(p.rank) * p.Tl + t;
    if (is_q) {
      const int o = h / Hql, hl = h - o * Hql;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.peers.base[o] + p.off_q) + (row * Hql + hl) * D;
      *reinterpret_cast<uint2*>(dst + 4 * lane) = raw;
    } else {
      const int hk = is_k ? h - p.Hq : h - p.Hq - p.Hk;
      const long long off = is_k ? p.off_k : p.off_v;
      for (int i = 0; i < p.rep; ++i) {
        const int r = hk * p.rep + i;
        const int o = r / Hkl, hl = r - o * Hkl;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.peers.base[o] + off) + (row * Hkl + hl) * D;
        *reinterpret_cast<uint2*>(dst + 4 * lane) = raw;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) last = (atomicAdd(p.done_counter, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last) {
    __threadfence_system();
    if (threadIdx.x < p.W) st_release_sys(reinterpret_cast<int*>(p.peers.base[threadIdx.x] + p.off_flags) + p.rank, p.epoch);
    if (threadIdx.x == 0) *p.done_counter = 0;
  }
}

struct UlyMoveParams {
  PeerTable peers;
  long long off_buf, off_flags;  // off_flags < 0: no flags (gather)
  __nv_bfloat16* local;          // [Tl, H, D] (source of a scatter, destination of a gather)
  long long Tl;
  int H, rep, W, rank, epoch;    // H: heads of `local`; destinations hold H * rep / W heads
  unsigned int* done_counter;
  const int* status;
};

__global__ void ulysses_scatter_kernel(const UlyMoveParams p) {
  constexpr int D = 128;
  const int lane = threadIdx.x & 31;
  const int Hl = p.H * p.rep / p.W;
  const long long total = p.Tl * p.H;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; gw < total; gw += nwarps) {
    const long long t = gw / p.H;
    const int h = static_cast<int>(gw - t * p.H);
    const uint2 v = *reinterpret_cast<const uint2*>(p.local + gw * D + 4 * lane);
    const long long row = static_cast<long long>(p.rank) * p.Tl + t;
    for (int i = 0; i < p.rep; ++i) {
      const int r = h * p.rep + i;
      const int o = r / Hl, hl = r - o * Hl;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.peers.base[o] + p.off_buf) + (row * Hl + hl) * D;
      *reinterpret_cast<uint2*>(dst + 4 * lane) = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) last = (atomicAdd(p.done_counter, 1u) == gridDim.x - 1);
  __syncthreads();
  if (last) {
    __threadfence_system();
    if (threadIdx.x < p.W) st_release_sys(reinterpret_cast<int*>(p.peers.base[threadIdx.x] + p.off_flags) + p.rank, p.epoch);
    if (threadIdx.x == 0) *p.done_counter = 0;
  }
}

__global__ void ulysses_gather_kernel(const UlyMoveParams p) {
  constexpr int D = 128;
  const int lane = threadIdx.x & 31;
  const int Hl = p.H * p.rep / p.W;
  const long long total = p.Tl * p.H;
  const bool healthy = (p.status == nullptr) || (*p.status == 0);
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; gw < total; gw += nwarps) {
    const long long t = gw / p.H;
    const int h = static_cast<int>(gw - t * p.H);
    const long long row = static_cast<long long>(p.rank) * p.Tl + t;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    uint2 single = make_uint2(0u, 0u);
    if (healthy) {
      for (int i = 0; i < p.rep; ++i) {
        const int r = h * p.rep + i;
        const int o = r / Hl, hl = r - o * Hl;
        const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(p.peers.base[o] + p.off_buf) + (row * Hl + hl) * D;
        const uint2 v = *reinterpret_cast<const uint2*>(src + 4 * lane);
        if (p.rep == 1) {
          single = v;
        } else {
          const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y);
          acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
        }
      }
    }
    if (p.rep != 1) single = make_uint2(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]));
    *reinterpret_cast<uint2*>(p.local + gw * D + 4 * lane) = single;
  }
}

}  // namespace ttb

TTB_EXPORT int ttb_ulysses_qkv_scatter(const unsigned long long* peer_ptrs, long long off_q, long long off_k,
                                       long long off_v, long long off_flags, const void* qkv, long long ld,
                                       const void* wq, const void* wk, const float* cos_t, const float* sin_t,
                                       float* rstd_out, long long Tl, int Hq, int Hk, int rep, int W, int rank,
                                       int epoch, int use_norm, float eps, unsigned int* done_counter, int grid,
                                       void* stream) {
  using namespace ttb;
  if (W > MAX_RANKS || W < 1 || ld % 8 || Hq % W || (Hk * rep) % W || rep < 1) return 901;
  UlyQkvParams p{make_peers(peer_ptrs, W), off_q, off_k, off_v, off_flags, (const __nv_bfloat16*)qkv, ld,
                 (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, cos_t, sin_t, rstd_out, Tl, Hq, Hk, rep, W, rank,
                 epoch, use_norm, eps, done_counter};
  if (grid < 1) grid = 1;
  ulysses_qkv_scatter_kernel<<<grid, 256, 0, STREAM(stream)>>>(p);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_ulysses_move(const unsigned long long* peer_ptrs, long long off_buf, long long off_flags, void* local,
                                long long Tl, int H, int rep, int W, int rank, int epoch, unsigned int* done_counter,
                                const int* status, int gather, int grid, void* stream) {
  using namespace ttb;
  if (W > MAX_RANKS || W < 1 || (H * rep) % W || rep < 1) return 901;
  UlyMoveParams p{make_peers(peer_ptrs, W), off_buf, off_flags, (__nv_bfloat16*)local, Tl, H, rep, W, rank, epoch,
                  done_counter, status};
  if (grid < 1) grid = 1;
  if (gather)
    ulysses_gather_kernel<<<grid, 256, 0, STREAM(stream)>>>(p);
  else
    ulysses_scatter_kernel<<<grid, 256, 0, STREAM(stream)>>>(p);
  LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------------------
// Sharded-data-parallel collectives over peer memory (the all-gather of parameter shards and the reduce-scatter
// of gradients of one FSDP unit).  Both are PULL kernels on a slot of the symmetric buffer that has the same
// offset on every rank:
//   all-gather     : slot = [W][n] pieces; rank r has written piece r; the kernel copies every other piece from
//                    its owner's slot into the local slot.
//   reduce-scatter : slot = [W][n] gradient pieces (piece q is what rank q must reduce); the kernel computes
//                    out[i] = scale * sum_p slot_of(p)[rank][i] in fp32 (bf16 or fp32 pieces) - the cast, the
//                    averaging scale and the reduction in one pass over NVLink.
// Flags: `ready[src]` (peer src has filled its slot for this epoch) is waited on before the first remote load;
// `consumed[src]` is raised on every peer when this rank has finished reading, and the next writer of the slot
// waits for it (host side, stream-ordered).  Waits are bounded; after a timeout no remote memory is touched.
// The NCCL ring kernels these replace: torch FSDP2's all_gather_into_tensor / reduce_scatter_tensor calls under
// the reference's fully_shard units (engine/backends/fsdp2/backend.py:420-470 of the reference).
// ------------------------------------------------------------------------------------------------------------
namespace ttb {

struct PeerCollParams {
  PeerTable peers;
  long long off_data, off_ready, off_consumed;
  long long units;   // 16-byte units per piece
  int rank, W, epoch;
  unsigned long long budget_ns;
  float scale;
  void* out;         // reduce-scatter result (local memory), same element type as the pieces
  unsigned int* done_counter;
  int* status;
};

__device__ __forceinline__ bool coll_wait_ready(const PeerCollParams& p, unsigned site) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.W && static_cast<int>(threadIdx.x) != p.rank) {
    const int* f = reinterpret_cast<const int*>(p.peers.base[p.rank] + p.off_ready) + threadIdx.x;
    if (!wait_flag(f, p.epoch, p.budget_ns, site, threadIdx.x, p.status)) s_ok = 0;
  }
  __syncthreads();
  return s_ok != 0;
}

__device__ __forceinline__ void coll_signal_consumed(const PeerCollParams& p) {
  __shared__ unsigned s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(p.done_counter, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < p.W)
      st_release_sys(reinterpret_cast<int*>(p.peers.base[threadIdx.x] + p.off_consumed) + p.rank, p.epoch);
    if (threadIdx.x == 0) *p.done_counter = 0;
  }
}

__global__ void __launch_bounds__(512) peer_allgather_kernel(const PeerCollParams p) {
  if (coll_wait_ready(p, 7)) {
    const long long total = p.units * (p.W - 1);
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    uint4* mine = reinterpret_cast<uint4*>(p.peers.base[p.rank] + p.off_data);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += 4 * stride) {
      uint4 v[4];
      long long at[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long ii = i + u * stride;
        at[u] = -1;
        if (ii < total) {
          const int j = static_cast<int>(ii / p.units);
          const int peer = (p.rank + 1 + j) % p.W;
          at[u] = static_cast<long long>(peer) * p.units + (ii - j * p.units);
          v[u] = __ldcg(reinterpret_cast<const uint4*>(p.peers.base[peer] + p.off_data) + at[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (at[u] >= 0) mine[at[u]] = v[u];
    }
  }
  coll_signal_consumed(p);
}

template <bool BF16>
__device__ __forceinline__ void rs_accumulate(float (&acc)[8], const uint4& v) {
  if (BF16) {
    const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), d = unpack_bf16(v.w);
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
    acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
  } else {
    acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
  }
}

// Each thread reduces RS_UNROLL 16-byte units at once and keeps RS_UNROLL x 2 remote loads in flight: one load per
// thread is latency-bound on NVLink (about 170 GB/s with 48 CTAs on two GPUs, against 480 GB/s with the loads batched).
constexpr int RS_UNROLL = 4;

template <bool BF16>
__global__ void __launch_bounds__(512) peer_reduce_scatter_kernel(const PeerCollParams p) {
  if (coll_wait_ready(p, 8)) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long piece = static_cast<long long>(p.rank) * p.units;
    for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < p.units;
         i0 += RS_UNROLL * stride) {
      float acc[RS_UNROLL][8];
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
      for (int j0 = 0; j0 < p.W; j0 += 2) {
        uint4 v[RS_UNROLL][2];
#pragma unroll
        for (int u = 0; u < RS_UNROLL; ++u) {
          const long long i = i0 + u * stride;
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            if (i < p.units && j0 + jj < p.W) {
              const int peer = (p.rank + j0 + jj) % p.W;
              v[u][jj] = __ldcg(reinterpret_cast<const uint4*>(p.peers.base[peer] + p.off_data) + piece + i);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < RS_UNROLL; ++u) {
          const long long i = i0 + u * stride;
#pragma unroll
          for (int jj = 0; jj < 2; ++jj)
            if (i < p.units && j0 + jj < p.W) rs_accumulate<BF16>(acc[u], v[u][jj]);
        }
      }
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i >= p.units) continue;
        const float* a = acc[u];
        uint4 o;
        if (BF16) {
          o.x = pack_bf16(a[0] * p.scale, a[1] * p.scale); o.y = pack_bf16(a[2] * p.scale, a[3] * p.scale);
          o.z = pack_bf16(a[4] * p.scale, a[5] * p.scale); o.w = pack_bf16(a[6] * p.scale, a[7] * p.scale);
        } else {
          o.x = __float_as_uint(a[0] * p.scale); o.y = __float_as_uint(a[1] * p.scale);
          o.z = __float_as_uint(a[2] * p.scale); o.w = __float_as_uint(a[3] * p.scale);
        }
        reinterpret_cast<uint4*>(p.out)[i] = o;
      }
    }
  }
  coll_signal_consumed(p);
}

}  // namespace ttb

// kind: 0 = all-gather (any element type, `units` 16-byte units per piece), 1 = reduce-scatter of fp32 pieces,
// 2 = reduce-scatter of bf16 pieces.  The caller has already raised its own `ready` flag (ttb_flag_signal) in
// stream order after filling the slot.
TTB_EXPORT int ttb_peer_collective(const unsigned long long* peer_ptrs, long long off_data, long long off_ready,
                                   long long off_consumed, long long units, int rank, int W, int epoch,
                                   long long budget_ms, float scale, void* out, unsigned int* done_counter, int* status,
                                   int kind, int grid, void* stream) {
  using namespace ttb;
  if (W > MAX_RANKS || W < 2 || units < 0 || off_data % 16) return 901;
  if (kind != 0 && (out == nullptr || reinterpret_cast<unsigned long long>(out) % 16)) return 903;
  PeerCollParams p{make_peers(peer_ptrs, W), off_data, off_ready, off_consumed, units, rank, W, epoch,
                   static_cast<unsigned long long>(budget_ms) * 1000000ull, scale, out, done_counter, status};
  if (grid < 1) grid = 1;
  if (kind == 0)
    peer_allgather_kernel<<<grid, 512, 0, STREAM(stream)>>>(p);
  else if (kind == 1)
    peer_reduce_scatter_kernel<false><<<grid, 512, 0, STREAM(stream)>>>(p);
  else
    peer_reduce_scatter_kernel<true><<<grid, 512, 0, STREAM(stream)>>>(p);
  LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------------------
// One host call per direction of an expert-parallel layer.  The kernels are the ones above (and the permutation
// helpers of moe.cu); launching them from one entry point only removes host work: the Python side of a 48-layer step
// made ~1000 separate calls for these sequences and the step is host-bound from two GPUs on.
// ------------------------------------------------------------------------------------------------------------
extern "C" int ttb_perm_rank(const int* idx, long long N, int E, const int* base, int* row_of, void* stream);
extern "C" int ttb_perm_zero_pad(void* dst, long long ldd, const int* counts, const int* seg_start, float* row_val, int E,
                                 int H, void* stream);

struct EpDispatchArgs {
  const unsigned long long* peer_ptrs;
  long long off_counts, off_flags_counts, off_rows, off_vals, off_flags_rows;
  const int* counts;       // [E] this rank's routing histogram
  const int* expert;       // [N] expert of every (token, slot) entry
  const void* src;         // [T, H] bf16 rows
  long long lds;
  const float* val;        // [N] routing weights or null
  void* recv_rows_local;   // this rank's receive buffer (for zeroing the padding rows)
  float* recv_vals_local;
  int* seg_start; int* recv_counts; int* tile_group; int* dest_base; int* dest_row;   // outputs
  unsigned int* done_counter;
  int* status;
  long long N, cap_rows, budget_ms;
  int rank, W, E, k, H, m_tiles_cap, epoch_counts, epoch_rows, grid, exchange;   // exchange = 0: tables are given
};

// forward dispatch (exchange = 1): counts exchange -> destination rows -> zero the padding -> scatter -> landed wait.
// backward of combine (exchange = 0): zero the padding -> scatter -> landed wait, with the forward's tables.
TTB_EXPORT int ttb_ep_dispatch_all(const EpDispatchArgs* a, void* stream) {
  int r;
  const int El = a->E / a->W;
  if (a->exchange) {
    r = ttb_ep_exchange(a->peer_ptrs, a->off_counts, a->off_flags_counts, a->counts, a->rank, a->W, a->E, a->epoch_counts,
                        a->budget_ms, a->m_tiles_cap, a->seg_start, a->recv_counts, a->tile_group, a->dest_base, a->status,
                        stream);
    if (r) return r;
    r = ttb_perm_rank(a->expert, a->N, a->E, a->dest_base, a->dest_row, stream);
    if (r) return r;
  }
  r = ttb_perm_zero_pad(a->recv_rows_local, a->H, a->recv_counts, a->seg_start, a->recv_vals_local, El, a->H, stream);
  if (r) return r;
  r = ttb_ep_scatter(a->peer_ptrs, a->off_rows, a->off_vals, a->off_flags_rows, a->src, a->lds, a->expert, a->dest_row, a->val,
                     a->N, a->k, a->H, El, a->rank, a->W, a->epoch_rows, a->cap_rows, a->done_counter, a->status, a->grid,
                     stream);
  if (r) return r;
  return ttb_flag_wait(a->peer_ptrs, a->off_flags_rows, a->rank, a->W, a->epoch_rows, a->budget_ms, a->status, stream);
}

// publish "my output rows are ready" -> wait for every owner -> pull and sum the k rows of every token
// (+ optionally the per-entry scalars, for the routing-weight gradient).
TTB_EXPORT int ttb_ep_combine_all(const unsigned long long* peer_ptrs, long long off_rows, long long off_vals,
                                  long long off_flags, const int* expert, const int* dest_row, const void* residual,
                                  long long ldr, void* out, long long ldo, float* vals_out, long long T, int k, int H,
                                  int El, int rank, int W, int epoch, long long budget_ms, long long cap_rows, int* status,
                                  void* stream) {
  int r = ttb_flag_signal(peer_ptrs, off_flags, rank, W, epoch, stream);
  if (r) return r;
  r = ttb_flag_wait(peer_ptrs, off_flags, rank, W, epoch, budget_ms, status, stream);
  if (r) return r;
  r = ttb_ep_gather(peer_ptrs, off_rows, expert, dest_row, nullptr, residual, ldr, out, ldo, T, k, H, El, W, cap_rows, status,
                    stream);
  if (r || vals_out == nullptr) return r;
  return ttb_ep_gather_vals(peer_ptrs, off_vals, expert, dest_row, vals_out, T * k, El, W, cap_rows, status, stream);
}


// ============================================================================================================
// Expert-parallel exchange fused into the grouped GEMMs (gemm.cu: push prologue, scatter epilogue).  What is left
// outside the GEMM kernels:
//   ttb_ep_prepare : counts exchange + layout tables + send order (forward only), destination rows, padding rows of
//                    the receive buffer zeroed with tag -1, progress counters cleared.  One host call.
//   ttb_ep_save    : copy of the rows that landed (device-side row count) for the backward pass.
//   ttb_ep_ksum    : waits (bounded) for every owner's "rows returned" flag, then out[t] = sum_j ret[t*k+j] (+ residual).
// ============================================================================================================
namespace ttb {

__global__ void ep_save_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const float* __restrict__ vsrc,
                                    float* __restrict__ vdst, const int* __restrict__ seg_start, int El, int vec,
                                    long long cap_rows) {
  long long rows = seg_start[El];
  if (rows > cap_rows) rows = cap_rows;
  const long long total = rows * vec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) dst[i] = src[i];
  if (vsrc)
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < rows; i += stride) vdst[i] = vsrc[i];
}

struct EpKsumParams {
  PeerTable peers;
  long long off_ret, off_ret_flags;
  const __nv_bfloat16* residual;
  long long ldr;
  __nv_bfloat16* out;
  long long ldo;
  int k, H, W, rank, epoch;
  unsigned long long budget_ns;
  int* status;
};

__global__ void ep_ksum_kernel(const EpKsumParams p) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < p.W) {
    const int* f = reinterpret_cast<const int*>(p.peers.base[p.rank] + p.off_ret_flags) + threadIdx.x;
    if (!wait_flag(f, p.epoch, p.budget_ns, 10, threadIdx.x, p.status)) s_ok = 0;
  }
  __syncthreads();
  const bool healthy = s_ok != 0;
  const long long t = blockIdx.x;
  const __nv_bfloat16* ret = reinterpret_cast<const __nv_bfloat16*>(p.peers.base[p.rank] + p.off_ret);
  for (int c = threadIdx.x * 8; c < p.H; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (healthy) {
      for (int j = 0; j < p.k; ++j) {
        const uint4 u = __ldcg(reinterpret_cast<const uint4*>(ret + (t * p.k + j) * p.H + c));
        float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
        acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
      }
    }
    if (p.residual) {
      const uint4 u = *reinterpret_cast<const uint4*>(p.residual + t * p.ldr + c);
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o4;
    o4.x = pack_bf16(acc[0], acc[1]); o4.y = pack_bf16(acc[2], acc[3]);
    o4.z = pack_bf16(acc[4], acc[5]); o4.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(p.out + t * p.ldo + c) = o4;
  }
}

}  // namespace ttb

extern "C" int ttb_perm_rank_order(const int* idx, long long N, int E, const int* base, int* row_of, const int* order_base,
                                   int* order, void* stream);
extern "C" int ttb_perm_zero_pad_tags(void* dst, long long ldd, const int* counts, const int* seg_start, float* row_val,
                                      int* row_tag, int* zero_ints, int n_zero, int E, int H, void* stream);

struct EpPrepareArgs {
  const unsigned long long* peer_ptrs;
  long long off_counts, off_flags_counts;
  const int* counts;        // [E] this rank's routing histogram
  const int* expert;        // [N]
  void* recv_rows_local;    // this rank's receive buffer: rows, scalars, tags
  float* recv_vals_local;
  int* recv_tags_local;
  int* seg_start; int* recv_counts; int* tile_group; int* dest_base; int* dest_row; int* send_base; int* order;   // tables
  int* sent;                // [E + 1] progress counters of the push warps (rows per expert, next chunk)
  int* status;
  long long N, budget_ms;
  int rank, W, E, H, m_tiles_cap, epoch_counts, exchange;   // exchange = 0: the tables of the forward pass are given
};

TTB_EXPORT int ttb_ep_prepare(const EpPrepareArgs* a, void* stream) {
  using namespace ttb;
  if (a->W > MAX_RANKS || a->W < 1 || a->E % a->W) return 901;
  const int El = a->E / a->W;
  int r;
  if (a->exchange) {
    const size_t sh = static_cast<size_t>(a->W) * a->E * 4 + static_cast<size_t>(a->W) * (El + 1) * 4;
    if (sh > 48 * 1024) return 902;
    EpExchangeParams p{make_peers(a->peer_ptrs, a->W), a->off_counts, a->off_flags_counts, a->counts, a->rank, a->W, a->E,
                       a->epoch_counts, static_cast<unsigned long long>(a->budget_ms) * 1000000ull, a->m_tiles_cap,
                       a->seg_start, a->recv_counts, a->tile_group, a->dest_base, a->status, a->send_base};
    ep_exchange_kernel<<<1, 256, sh, STREAM(stream)>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return 400 + (int)e;
    r = ttb_perm_rank_order(a->expert, a->N, a->E, a->dest_base, a->dest_row, a->send_base, a->order, stream);
    if (r) return r;
  }
  return ttb_perm_zero_pad_tags(a->recv_rows_local, a->H, a->recv_counts, a->seg_start, a->recv_vals_local,
                                a->recv_tags_local, a->sent, a->E + 1, El, a->H, stream);
}

TTB_EXPORT int ttb_ep_save(const void* src, void* dst, const float* vsrc, float* vdst, const int* seg_start, int El, int H,
                           long long cap_rows, int grid, void* stream) {
  if (H % 8) return 901;
  if (grid < 1) grid = 1;
  ttb::ep_save_rows_kernel<<<grid, 256, 0, STREAM(stream)>>>((const uint4*)src, (uint4*)dst, vsrc, vdst, seg_start, El, H / 8,
                                                           cap_rows);
  LAUNCH_RET();
}

TTB_EXPORT int ttb_ep_ksum(const unsigned long long* peer_ptrs, long long off_ret, long long off_ret_flags, const void* residual,
                           long long ldr, void* out, long long ldo, long long T, int k, int H, int W, int rank, int epoch,
                           long long budget_ms, int* status, void* stream) {
  using namespace ttb;
  if (W > MAX_RANKS || W < 1 || H % 8 || ldo % 8 || (residual && ldr % 8)) return 901;
  if (T == 0) return 0;
  EpKsumParams p{make_peers(peer_ptrs, W), off_ret, off_ret_flags, (const __nv_bfloat16*)residual, ldr, (__nv_bfloat16*)out,
                 ldo, k, H, W, rank, epoch, static_cast<unsigned long long>(budget_ms) * 1000000ull, status};
  int threads = H / 8;
  threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  ep_ksum_kernel<<<(unsigned)T, threads, 0, STREAM(stream)>>>(p);
  LAUNCH_RET();
}


// ============================================================================================================
// In-switch all-reduce of one symmetric fp32 buffer (NVLS multimem): rank r owns slice r of the buffer; it loads the
// SUM of that slice over all ranks with one `multimem.ld_reduce` per 16 bytes (the NVSwitch adds the W copies on the
// way), scales it and writes the result to every rank's buffer with one `multimem.st` (the switch replicates it).
// Per GPU that is 1/W of the buffer in and 1/W out instead of the 2 (W-1)/W of a ring.  `mc` is the multicast
// address of the buffer (same offset on every rank).  The caller brackets the kernel with the epoch-flag barrier
// (every rank has finished writing its gradients / every rank has finished storing its slice).
// Used for the flat gradient buffer of replicated decoder layers; the NCCL all-reduce it replaces is the one the
// reference issues per replicated parameter (engine/backends/fsdp2/backend.py:415-436 there).
// ============================================================================================================
namespace ttb {
__device__ __forceinline__ void mm_ld_reduce_v4(const float* addr, float& a, float& b, float& c, float& d) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(a), "=f"(b), "=f"(c), "=f"(d)
               : "l"(addr)
               : "memory");
}
__device__ __forceinline__ void mm_st_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Four independent 16-byte reductions in flight per thread: one `multimem.ld_reduce` is a round trip to the switch.
__global__ void __launch_bounds__(512) multimem_allreduce_f32_kernel(float* mc, long long first4, long long last4, float scale) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = first4 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < last4; i += 4 * stride) {
    float v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) mm_ld_reduce_v4(mc + 4 * (i + u * stride), v[u][0], v[u][1], v[u][2], v[u][3]);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      mm_st_v4(mc + 4 * (i + u * stride), v[u][0] * scale, v[u][1] * scale, v[u][2] * scale, v[u][3] * scale);
  }
  for (; i < last4; i += stride) {
    float a, b, c, d;
    mm_ld_reduce_v4(mc + 4 * i, a, b, c, d);
    mm_st_v4(mc + 4 * i, a * scale, b * scale, c * scale, d * scale);
  }
}
}  // namespace ttb

// `n` floats (multiple of 4) at multicast address `mc`; this rank reduces and broadcasts slice `rank` of `W`.
TTB_EXPORT int ttb_multimem_allreduce_f32(void* mc, long long n, int rank, int W, float scale, int grid, void* stream) {
  if (mc == nullptr || (reinterpret_cast<unsigned long long>(mc) & 15) || n < 0 || (n & 3) || W < 1 || rank < 0 || rank >= W)
    return 901;
  const long long n4 = n / 4;
  const long long per = (n4 + W - 1) / W;
  const long long first = per * rank < n4 ? per * rank : n4;
  const long long last = first + per < n4 ? first + per : n4;
  if (grid < 1) grid = 1;
  if (last > first)
    ttb::multimem_allreduce_f32_kernel<<<grid, 512, 0, STREAM(stream)>>>(reinterpret_cast<float*>(mc), first, last, scale);
  LAUNCH_RET();
}
