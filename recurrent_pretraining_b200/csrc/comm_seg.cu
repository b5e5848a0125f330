// Tensor-table forms of the sharded data-parallel step.
//
// Ownership is per tensor: rank q owns elements [q * per, min(numel, (q + 1) * per)) of every tensor of a flat
// optimizer group (`per` is a whole number of rows where the shape allows, so that a row-sharded weight can also be
// gathered by the GEMM that consumes it).  A bucket of tensors is described by ONE small table passed by value, from
// which a kernel derives any rank's segments; one launch then covers all tensors of the bucket:
//
//   rs_tab_kernel      reduce-scatter of fp32 gradients over the owner's segments (+ squared-norm partial), with the
//                      peers' "bucket ready" flags awaited inside the kernel (bounded), so that a bucket can be reduced
//                      on a side stream while the backward pass of the remaining layers is still running
//   signal_kernel      publishes "my gradients of bucket b are complete" to every peer
//   opt_stats_kernel   per-tensor sum of g^2 / max(v', eps^2) for the update clipping of ELLISAdam
//   opt_tab_kernel     AdamW / ELLISAdam (running init, atan2 update, decoupled decay, per-tensor update clipping) on
//                      the owner's segments; writes the bf16 compute copy to every rank given (all peers in the
//                      replicated mode, only the owner in the parameter-sharded mode)
//   ag_tab_kernel      pull all-gather of the bf16 compute copies: every other rank's segments are read from that
//                      rank's buffer into the same offsets of the local one
//
// Peers are touched by plain loads and stores only.  A wait that runs out sets the status word, poisons the norm (the
// update kernels skip a step whose norm is not finite) and the kernel returns.
#include "common.cuh"

namespace b200 {

constexpr int MAX_RANKS_T = 16;
constexpr int MAX_TT = 48;

struct PeerPtrsT {
  void* p[MAX_RANKS_T];
};

struct TensorTable {
  int n;                     // tensors in this launch
  int n_ranks;
  long long off[MAX_TT];     // element offset of the tensor inside the group's flat buffers
  long long numel[MAX_TT];
  long long per[MAX_TT];     // elements owned by each rank
  long long soff[MAX_TT];    // offset of this rank's segment inside its concatenated state (m, v, sharded master)
  int stat[MAX_TT];          // index of the tensor in the per-tensor statistics array
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_sys_f4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_sys_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Segments of rank q in shared memory: start (element offset in the flat buffer), prefix (elements before the segment
// in the launch-local concatenation; prefix[n] = total).  Called by the whole CTA.
struct SegSmem {
  long long start[MAX_TT];
  long long prefix[MAX_TT + 1];
};
__device__ __forceinline__ void build_segments(const TensorTable& tb, int q, SegSmem& s) {
  if (threadIdx.x == 0) {
    long long acc = 0;
    for (int t = 0; t < tb.n; ++t) {
      long long lo = static_cast<long long>(q) * tb.per[t];
      if (lo > tb.numel[t]) lo = tb.numel[t];
      long long hi = lo + tb.per[t];
      if (hi > tb.numel[t]) hi = tb.numel[t];
      s.start[t] = tb.off[t] + lo;
      s.prefix[t] = acc;
      acc += hi - lo;
    }
    s.prefix[tb.n] = acc;
  }
  __syncthreads();
}
// flat element offset of concatenated element `e`; `cur` is a cursor that only moves forward
__device__ __forceinline__ long long locate(const SegSmem& s, int n, long long e, int& cur) {
  while (cur + 1 < n && e >= s.prefix[cur + 1]) ++cur;
  return s.start[cur] + (e - s.prefix[cur]);
}

// Publishes `epoch` in slot [rank] of every rank's flag array (one thread per peer).
__global__ void signal_kernel(const __grid_constant__ PeerPtrsT flags, int rank, int N, uint32_t epoch) {
  const int i = threadIdx.x;
  if (i < N) {
    __threadfence_system();
    st_release_sys_u32(reinterpret_cast<uint32_t*>(flags.p[i]) + rank, epoch);
  }
}

// Waits (bounded) until every rank's flag in this rank's array reached `epoch`.  Whole CTA; returns false on time-out.
__device__ __forceinline__ bool wait_flags(const uint32_t* mine, int N, uint32_t epoch, unsigned long long timeout_ns,
                                           int* err) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < N) {
    const unsigned long long t0 = globaltimer_ns();
    while (true) {
      const uint32_t v = ld_acquire_sys_u32(mine + threadIdx.x);
      if (static_cast<int32_t>(v - epoch) >= 0) break;
      if (globaltimer_ns() - t0 > timeout_ns) {
        s_fail = 1;
        if (err) atomicCAS(err, 0, ERR_WAIT_PEER_FLAG);
        break;
      }
      __nanosleep(128);
    }
  }
  __syncthreads();
  return s_fail == 0;
}

__device__ __forceinline__ void block_add(float v, float* red16, float* dst) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red16[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red16[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(dst, t);
  }
}

// own[seg] = sum over ranks of buf_q[seg] for every segment of `rank`; *sumsq += squared norm of the result.
// epoch != 0: wait until all ranks published `epoch` in this rank's flag array (signal != 0: publish first).
template <int N, int U>
__global__ void __launch_bounds__(512)
rs_tab_kernel(const __grid_constant__ PeerPtrsT bufs, int rank, const __grid_constant__ TensorTable tb, float* sumsq,
              const __grid_constant__ PeerPtrsT flags, uint32_t epoch, int signal, unsigned long long timeout_ns,
              int* err) {
  __shared__ SegSmem seg;
  __shared__ float red[16];
  build_segments(tb, rank, seg);
  if (epoch != 0) {
    if (signal && blockIdx.x == 0 && threadIdx.x < N) {
      __threadfence_system();
      st_release_sys_u32(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + rank, epoch);
    }
    if (!wait_flags(reinterpret_cast<const uint32_t*>(flags.p[rank]), N, epoch, timeout_ns, err)) {
      if (sumsq && blockIdx.x == 0 && threadIdx.x == 0) *sumsq = __int_as_float(0x7fc00000);
      return;
    }
  }
  float* own = reinterpret_cast<float*>(bufs.p[rank]);
  const float* peer[N];
#pragma unroll
  for (int q = 0; q < N; ++q) peer[q] = reinterpret_cast<const float*>(bufs.p[(q + rank) % N]);
  const long long nvec = seg.prefix[tb.n] >> 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float ss = 0.f;
  int cur = 0;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += U * stride) {
    float4 v[U][N];
    long long at[U];
    int c = cur;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long iv = i + u * stride;
      at[u] = -1;
      if (iv < nvec) {
        at[u] = locate(seg, tb.n, iv << 2, c);
        if (u == 0) cur = c;
#pragma unroll
        for (int q = 0; q < N; ++q) v[u][q] = ld_sys_f4(reinterpret_cast<const float4*>(peer[q] + at[u]));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (at[u] >= 0) {
        float4 a = v[u][0];
#pragma unroll
        for (int q = 1; q < N; ++q) { a.x += v[u][q].x; a.y += v[u][q].y; a.z += v[u][q].z; a.w += v[u][q].w; }
        *reinterpret_cast<float4*>(own + at[u]) = a;
        ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      }
    }
  }
  if (sumsq) block_add(ss, red, sumsq);
}

// Pull all-gather of 16-byte units (bf16 compute copies): blockIdx.y selects the peer (rank + 1 + y) % N.
__global__ void __launch_bounds__(512)
ag_tab_kernel(const __grid_constant__ PeerPtrsT bufs, int rank, int N, const __grid_constant__ TensorTable tb) {
  __shared__ SegSmem seg;
  const int q = (rank + 1 + blockIdx.y) % N;
  build_segments(tb, q, seg);
  const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(bufs.p[q]);
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(bufs.p[rank]);
  const long long nvec = seg.prefix[tb.n] >> 3;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int U = 4;
  int cur = 0;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += U * stride) {
    uint4 v[U];
    long long at[U];
    int c = cur;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long iv = i + u * stride;
      at[u] = -1;
      if (iv < nvec) {
        at[u] = locate(seg, tb.n, iv << 3, c);
        if (u == 0) cur = c;
        v[u] = ld_sys_u4(reinterpret_cast<const uint4*>(src + at[u]));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (at[u] >= 0) *reinterpret_cast<uint4*>(dst + at[u]) = v[u];
  }
}

struct OptArgs {
  float lr, beta1, beta2, eps, decay;   // decay: factor applied to the parameter (1 - lr * wd, or 1 - lr / lr0 * wd)
  float bc1, bc2;                       // 1 - beta^t
  float max_norm, grad_scale;
  int atan2_mode, update_clip, state_init, zero_grad;
  int n_push, push_master, master_sharded, n_ranks;
  int max_ctas;                         // 0: as many CTAs as the work fills; else a cap (an update that runs beside the
                                        // next step's forward pass leaves the SMs to its GEMMs)
};

__device__ __forceinline__ float clip_scale(const float* gnorm_sq, const OptArgs& a, bool& skip) {
  float clip = 1.f;
  skip = false;
  if (gnorm_sq) {
    const float gn = sqrtf(*gnorm_sq) * a.grad_scale;
    if (!isfinite(gn)) skip = true;
    else if (a.max_norm > 0.f) clip = fminf(1.f, a.max_norm / (gn + 1e-6f));
  }
  return a.grad_scale * clip;
}

// stats[tb.stat[t]] += sum over this rank's segment of tensor t (= blockIdx.y) of g^2 / max(v', eps^2), g the clipped
// and scaled gradient and v' the second moment after this step's update (not stored here).
__global__ void __launch_bounds__(256)
opt_stats_kernel(const float* __restrict__ g, const float* __restrict__ v, const __grid_constant__ TensorTable tb,
                 int rank, const float* __restrict__ gnorm_sq, OptArgs a, float* __restrict__ stats) {
  __shared__ float red[16];
  const int t = blockIdx.y;
  long long lo = static_cast<long long>(rank) * tb.per[t];
  if (lo > tb.numel[t]) lo = tb.numel[t];
  long long hi = lo + tb.per[t];
  if (hi > tb.numel[t]) hi = tb.numel[t];
  bool skip;
  const float gs = clip_scale(gnorm_sq, a, skip);
  if (skip || hi <= lo) return;
  const float4* gp = reinterpret_cast<const float4*>(g + tb.off[t] + lo);
  const float4* vp = reinterpret_cast<const float4*>(v + tb.soff[t]);
  const long long nvec = (hi - lo) >> 2;
  const float e2 = a.eps * a.eps;
  float s = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 gv = gp[i];
    float4 vv = a.state_init ? make_float4(0.f, 0.f, 0.f, 0.f) : vp[i];
    const float gg[4] = {gv.x * gs, gv.y * gs, gv.z * gs, gv.w * gs};
    const float vo[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g2 = gg[j] * gg[j];
      const float vn = a.state_init ? g2 : a.beta2 * vo[j] + (1.f - a.beta2) * g2;
      s += g2 / fmaxf(vn, e2);
    }
  }
  block_add(s, red, stats + tb.stat[t]);
}

// The update on this rank's segments.  p: fp32 master (full buffer, or the concatenated shard when master_sharded);
// g: full fp32 gradient buffer (already reduced on the segments); m, v: concatenated state; shadows / masters: the
// bf16 compute copy (and, for the group that the kernels read in fp32, the master) of every rank that receives the
// result; stats: per-tensor statistics arrays of all ranks (update clipping), summed here.
__global__ void __launch_bounds__(256)
opt_tab_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
               const __grid_constant__ PeerPtrsT shadows, const __grid_constant__ PeerPtrsT masters,
               const __grid_constant__ PeerPtrsT stats, const __grid_constant__ TensorTable tb, int rank,
               const float* __restrict__ gnorm_sq, OptArgs a) {
  __shared__ SegSmem seg;
  __shared__ float s_step[MAX_TT];
  build_segments(tb, rank, seg);
  if (threadIdx.x < tb.n) {
    float step = a.lr;
    if (a.update_clip) {
      float tot = 0.f;
      for (int q = 0; q < a.n_ranks; ++q) tot += *(reinterpret_cast<const volatile float*>(stats.p[q]) + tb.stat[threadIdx.x]);
      const float rms = sqrtf(tot / static_cast<float>(tb.numel[threadIdx.x]));
      step = a.lr / fmaxf(rms, 1.f);
    }
    s_step[threadIdx.x] = step / a.bc1;
  }
  __syncthreads();
  bool skip;
  const float gs = clip_scale(gnorm_sq, a, skip);
  const float inv_sqrt_bc2 = rsqrtf(a.bc2);
  const float e2 = a.eps * a.eps;
  const long long nvec = seg.prefix[tb.n] >> 2;
  int cur = 0;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = i << 2;
    const long long at = locate(seg, tb.n, e, cur);
    const long long st = tb.soff[cur] + (e - seg.prefix[cur]);
    float* pp_ptr = a.master_sharded ? p + st : p + at;
    float4 pv = *reinterpret_cast<float4*>(pp_ptr);
    if (!skip) {
      const float4 gv = *reinterpret_cast<const float4*>(g + at);
      float4 mv = a.state_init ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<float4*>(m + st);
      float4 vv = a.state_init ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<float4*>(v + st);
      float* pp = reinterpret_cast<float*>(&pv);
      const float* gp = reinterpret_cast<const float*>(&gv);
      float* mp = reinterpret_cast<float*>(&mv);
      float* vp = reinterpret_cast<float*>(&vv);
      const float step = s_step[cur];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = gp[j] * gs;
        if (a.state_init) { mp[j] = gj; vp[j] = gj * gj; }
        mp[j] = mp[j] + (1.f - a.beta1) * (gj - mp[j]);
        vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gj * gj;
        if (a.update_clip) vp[j] = fmaxf(vp[j], e2);
        float pj = pp[j] * a.decay;
        if (a.atan2_mode) pj -= step * atan2f(mp[j], sqrtf(vp[j]) * inv_sqrt_bc2);
        else pj -= step * mp[j] / (sqrtf(vp[j]) * inv_sqrt_bc2 + a.eps);
        pp[j] = pj;
      }
      *reinterpret_cast<float4*>(pp_ptr) = pv;
      *reinterpret_cast<float4*>(m + st) = mv;
      *reinterpret_cast<float4*>(v + st) = vv;
    }
    if (a.zero_grad) *reinterpret_cast<float4*>(g + at) = make_float4(0.f, 0.f, 0.f, 0.f);
    uint2 o;
    o.x = pack_bf16x2(pv.x, pv.y);
    o.y = pack_bf16x2(pv.z, pv.w);
    for (int q = 0; q < a.n_push; ++q) {
      if (shadows.p[q]) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(shadows.p[q]) + at) = o;
      if (a.push_master && masters.p[q]) *reinterpret_cast<float4*>(reinterpret_cast<float*>(masters.p[q]) + at) = pv;
    }
  }
}

// Cross-rank barrier on one flag slot that also adds up `n_sum` floats per rank (norm partial, ...): out[j] = sum over
// ranks of partial_q[j].  A time-out makes every out[j] NaN.
__global__ void barrier_sum_kernel(const __grid_constant__ PeerPtrsT flags, int rank, int N, uint32_t epoch,
                                   unsigned long long timeout_ns, const __grid_constant__ PeerPtrsT partials, int n_sum,
                                   float* out, int* err) {
  if (threadIdx.x < N) {
    __threadfence_system();
    st_release_sys_u32(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + rank, epoch);
  }
  const bool ok = wait_flags(reinterpret_cast<const uint32_t*>(flags.p[rank]), N, epoch, timeout_ns, err);
  if (out && threadIdx.x < n_sum) {
    float s = 0.f;
    if (ok) {
      for (int q = 0; q < N; ++q) s += *(reinterpret_cast<const volatile float*>(partials.p[q]) + threadIdx.x);
    } else {
      s = __int_as_float(0x7fc00000);
    }
    out[threadIdx.x] = s;
  }
}

}  // namespace b200

using namespace b200;

static PeerPtrsT mk(void* const* host_ptrs, int N, long long byte_offset = 0) {
  PeerPtrsT pp;
  for (int i = 0; i < MAX_RANKS_T; ++i)
    pp.p[i] = (i < N && host_ptrs && host_ptrs[i]) ? static_cast<char*>(host_ptrs[i]) + byte_offset : nullptr;
  return pp;
}

static int check_table(const TensorTable* tb, int vec) {
  if (!tb || tb->n < 0 || tb->n > MAX_TT) return -4;
  for (int t = 0; t < tb->n; ++t)
    if ((tb->off[t] % vec) || (tb->per[t] % vec) || (tb->numel[t] % vec) || (tb->soff[t] % 4)) return -3;
  return 0;
}

static inline int grid_cap(long long nvec, int threads, int cap) {
  long long b = (nvec + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return static_cast<int>(b);
}

static long long owned_total(const TensorTable* tb, int q) {
  long long tot = 0;
  for (int t = 0; t < tb->n; ++t) {
    long long lo = static_cast<long long>(q) * tb->per[t];
    if (lo > tb->numel[t]) lo = tb->numel[t];
    long long hi = lo + tb->per[t];
    if (hi > tb->numel[t]) hi = tb->numel[t];
    tot += hi - lo;
  }
  return tot;
}

B200_API int b200_table_size() { return static_cast<int>(sizeof(TensorTable)); }
B200_API int b200_table_max() { return MAX_TT; }

B200_API int b200_signal(void* const* flag_ptrs, int rank, int N, unsigned int epoch, void* stream) {
  if (N > MAX_RANKS_T) return -1;
  signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(mk(flag_ptrs, N), rank, N, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

#define DISPATCH_NT(N_, CALL)                      \
  switch (N_) {                                    \
    case 1: { constexpr int NN = 1; CALL; break; } \
    case 2: { constexpr int NN = 2; CALL; break; } \
    case 3: { constexpr int NN = 3; CALL; break; } \
    case 4: { constexpr int NN = 4; CALL; break; } \
    case 5: { constexpr int NN = 5; CALL; break; } \
    case 6: { constexpr int NN = 6; CALL; break; } \
    case 7: { constexpr int NN = 7; CALL; break; } \
    case 8: { constexpr int NN = 8; CALL; break; } \
    default: return -1;                            \
  }

// Reduce-scatter of the fp32 gradients of one bucket (see rs_tab_kernel).  ctas <= 0 picks 296.
B200_API int b200_rs_table(void* const* buf_ptrs, int rank, int N, const void* table, float* sumsq,
                           void* const* flag_ptrs, unsigned int epoch, int signal, int timeout_ms, int ctas, int* err,
                           void* stream) {
  const TensorTable* tb = reinterpret_cast<const TensorTable*>(table);
  if (int rc = check_table(tb, 4)) return rc;
  const long long nvec = owned_total(tb, rank) >> 2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (nvec == 0 && epoch == 0) return 0;
  const int grid = grid_cap(nvec, 512 * 2, ctas > 0 ? ctas : 296);
  const PeerPtrsT bp = mk(buf_ptrs, N), fp = mk(flag_ptrs, N);
  const unsigned long long to = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  DISPATCH_NT(N, (rs_tab_kernel<NN, (NN <= 4 ? 4 : 2)><<<grid, 512, 0, st>>>(bp, rank, *tb, sumsq, fp, epoch, signal, to, err)))
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Pull the bf16 segments of every other rank into the local buffer.
B200_API int b200_ag_table(void* const* buf_ptrs, int rank, int N, const void* table, int ctas, void* stream) {
  const TensorTable* tb = reinterpret_cast<const TensorTable*>(table);
  if (int rc = check_table(tb, 8)) return rc;
  if (N < 2) return 0;
  long long most = 0;
  for (int q = 0; q < N; ++q) {
    const long long o = owned_total(tb, q);
    if (o > most) most = o;
  }
  if (most == 0) return 0;
  int cap = (ctas > 0 ? ctas : 296) / (N - 1);
  if (cap < 1) cap = 1;
  const int per_peer = grid_cap(most >> 3, 512 * 4, cap);
  ag_tab_kernel<<<dim3(per_peer, N - 1), 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(mk(buf_ptrs, N), rank, N, *tb);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

struct OptHost {
  float lr, beta1, beta2, eps, decay, bc1, bc2, max_norm, grad_scale;
  int atan2_mode, update_clip, state_init, zero_grad, n_push, push_master, master_sharded, n_ranks, max_ctas;
};

B200_API int b200_opt_stats(const float* g, const float* v, const void* table, int rank, const float* gnorm_sq,
                            const void* opt, float* stats, void* stream) {
  const TensorTable* tb = reinterpret_cast<const TensorTable*>(table);
  if (int rc = check_table(tb, 4)) return rc;
  if (tb->n == 0) return 0;
  OptArgs a;
  static_assert(sizeof(OptArgs) == sizeof(OptHost), "argument block");
  memcpy(&a, opt, sizeof(a));
  opt_stats_kernel<<<dim3(64, tb->n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(g, v, *tb, rank, gnorm_sq, a, stats);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_opt_table(float* p, float* g, float* m, float* v, void* const* shadow_ptrs, void* const* master_ptrs,
                            void* const* stat_ptrs, const void* table, int rank, const float* gnorm_sq, const void* opt,
                            void* stream) {
  const TensorTable* tb = reinterpret_cast<const TensorTable*>(table);
  if (int rc = check_table(tb, 4)) return rc;
  OptArgs a;
  memcpy(&a, opt, sizeof(a));
  if (a.n_push > MAX_RANKS_T || a.n_ranks > MAX_RANKS_T) return -1;
  const long long nvec = owned_total(tb, rank) >> 2;
  if (nvec == 0) return 0;
  const int grid = grid_cap(nvec, 256, a.max_ctas > 0 ? a.max_ctas : 148 * 8);
  opt_tab_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      p, g, m, v, mk(shadow_ptrs, a.n_push), mk(master_ptrs, a.n_push), mk(stat_ptrs, a.n_ranks), *tb, rank, gnorm_sq, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Barrier on one flag slot; out[j] (j < n_sum <= 32) = sum over ranks of the floats at partial_ptrs[q][j].
B200_API int b200_barrier_sum(void* const* flag_ptrs, int rank, int N, unsigned int epoch, int timeout_ms,
                              void* const* partial_ptrs, int n_sum, float* out, int* err, void* stream) {
  if (N > MAX_RANKS_T || n_sum > 32) return -1;
  barrier_sum_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      mk(flag_ptrs, N), rank, N, epoch, static_cast<unsigned long long>(timeout_ms) * 1000000ull, mk(partial_ptrs, N),
      partial_ptrs ? n_sum : 0, partial_ptrs ? out : nullptr, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
