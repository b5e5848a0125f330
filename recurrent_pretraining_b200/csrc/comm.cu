// Gradient synchronisation over NVLink peer memory, written as plain CUDA kernels on symmetric buffers (every rank
// maps every other rank's buffer through CUDA IPC).  One process per GPU; ranks meet at flag barriers whose waits
// are bounded.  The data path of one optimizer step in data-parallel training is
//
//   barrier -> reduce-scatter (+ squared-norm partial) -> barrier (+ norm exchange) -> sharded AdamW that PUSHES the
//   bf16 compute copy of its slice to every rank -> barrier
//
// i.e. a two-shot all-reduce in which the second shot carries updated bf16 parameters instead of fp32 gradients:
// (N-1)/N * 4 bytes in and (N-1)/N * 2 bytes out per parameter instead of 2 * (N-1)/N * 4, with the update itself
// done once per parameter instead of N times.  Also here: a plain in-place all-reduce (one-shot for small buffers,
// two-shot otherwise) for the communication sweep and for callers that keep replicated optimizer state.
//
// Only ordinary peer loads/stores are used (ld.global.cg / st.global through the NVSwitch); no TMA multicast and no
// multimem instructions, so a rank that dies cannot fault its peers' GPUs.
#include "common.cuh"

namespace b200 {

constexpr int MAX_RANKS = 16;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Cross-rank barrier: thread i publishes `epoch` in slot [rank] of rank i's flag array and waits until slot [i] of
// its own array reaches `epoch`.  Optionally sums one float per rank (the squared-norm partials) after the wait.
// status: 0 ok, ERR_WAIT_PEER_FLAG after `timeout_ns` without the peer's flag.
__global__ void barrier_kernel(const __grid_constant__ PeerPtrs flags, int rank, int N, uint32_t epoch, unsigned long long timeout_ns,
                               const __grid_constant__ PeerPtrs partials, float* total_out, int* err) {
  __shared__ int ok_count;
  if (threadIdx.x == 0) ok_count = 0;
  __syncthreads();
  const int i = threadIdx.x;
  if (i < N) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[i]) + rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + i;
    const unsigned long long t0 = globaltimer_ns();
    bool ok = false;
    while (true) {
      const uint32_t v = ld_acquire_sys(mine);
      if (static_cast<int32_t>(v - epoch) >= 0) { ok = true; break; }
      if (globaltimer_ns() - t0 > timeout_ns) break;
      __nanosleep(64);
    }
    if (ok) atomicAdd(&ok_count, 1);
    else if (err) atomicCAS(err, 0, ERR_WAIT_PEER_FLAG);
  }
  __syncthreads();
  if (threadIdx.x == 0 && total_out) {
    float s = 0.f;
    if (ok_count == N) {
      for (int q = 0; q < N; ++q) s += *reinterpret_cast<volatile float*>(partials.p[q]);
    } else {
      s = __int_as_float(0x7fc00000);  // NaN: the optimizer kernel treats a non-finite norm as "skip the step"
    }
    *total_out = s;
  }
}

// In-place reduce-scatter of fp32: own[start .. start+count) = sum over ranks of buf_q[start .. start+count);
// *sumsq += sum of squares of the reduced values.  count % 4 == 0, pointers 16-byte aligned.
template <int N, int U>
__global__ void __launch_bounds__(512)
reduce_scatter_kernel(const __grid_constant__ PeerPtrs bufs, int rank, size_t start, size_t count, float* sumsq) {
  __shared__ float red[16];
  float4* own = reinterpret_cast<float4*>(reinterpret_cast<float*>(bufs.p[rank]) + start);
  const float4* peer[N];
#pragma unroll
  for (int q = 0; q < N; ++q) peer[q] = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(bufs.p[(q + rank) % N]) + start);
  float ss = 0.f;
  const size_t nvec = count >> 2;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // U independent vectors per thread per trip: U * (N - 1) remote 16-byte loads in flight per thread
  for (; i + (U - 1) * stride < nvec; i += U * stride) {
    float4 v[U][N];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int q = 0; q < N; ++q) v[u][q] = ld_peer_f4(peer[q] + i + u * stride);  // q = 0 is the local copy
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float4 a = v[u][0];
#pragma unroll
      for (int q = 1; q < N; ++q) { a.x += v[u][q].x; a.y += v[u][q].y; a.z += v[u][q].z; a.w += v[u][q].w; }
      own[i + u * stride] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  for (; i < nvec; i += stride) {
    float4 a = ld_peer_f4(peer[0] + i);
#pragma unroll
    for (int q = 1; q < N; ++q) {
      const float4 w = ld_peer_f4(peer[q] + i);
      a.x += w.x; a.y += w.y; a.z += w.z; a.w += w.w;
    }
    own[i] = a;
    ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  if (sumsq) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 16) {
      float t = red[threadIdx.x];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffu, t, o);
      if (threadIdx.x == 0) atomicAdd(sumsq, t);
    }
  }
}

// Pull all-gather of 16-byte units: own[slice q] = buf_q[slice q] for every q != rank, slices of `slice_vec` uint4.
__global__ void __launch_bounds__(512)
allgather_kernel(const __grid_constant__ PeerPtrs bufs, int rank, int N, size_t slice_vec, size_t total_vec) {
  uint4* own = reinterpret_cast<uint4*>(bufs.p[rank]);
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_vec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int q = static_cast<int>(i / slice_vec);
    if (q == rank || q >= N) continue;
    uint4 v;
    const uint4* src = reinterpret_cast<const uint4*>(bufs.p[q]) + i;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(src)
                 : "memory");
    own[i] = v;
  }
}

// Push all-gather: this rank's slice is written into every peer's buffer at the same offset (stores need no
// request/response round trip over NVLink, unlike the pull form above).
__global__ void __launch_bounds__(512)
allgather_push_kernel(const __grid_constant__ PeerPtrs bufs, int rank, int N, size_t slice_vec) {
  const uint4* src = reinterpret_cast<const uint4*>(bufs.p[rank]) + static_cast<size_t>(rank) * slice_vec;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < slice_vec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
    for (int q = 1; q < N; ++q) {
      const int dst = (rank + q) % N;
      reinterpret_cast<uint4*>(bufs.p[dst])[static_cast<size_t>(rank) * slice_vec + i] = v;
    }
  }
}

// One-shot all-reduce for small buffers: every rank reads all copies and writes the sum into `out` (its own,
// separate result buffer, so that no rank overwrites data a peer may still be reading).
template <int N>
__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(const __grid_constant__ PeerPtrs bufs, int rank, float* out, size_t count, float scale, float* sumsq) {
  __shared__ float red[16];
  float ss = 0.f;
  const size_t nvec = count >> 2;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < N; ++q) {
      const float4 v = ld_peer_f4(reinterpret_cast<const float4*>(bufs.p[(q + rank) % N]) + i);
      a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
    reinterpret_cast<float4*>(out)[i] = a;
    ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
  }
  if (sumsq) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 16) {
      float t = red[threadIdx.x];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffu, t, o);
      if (threadIdx.x == 0) atomicAdd(sumsq, t);
    }
  }
}

// bf16 -> fp32 variants for the communication sweep (bf16 buckets reduced in fp32)
template <int N>
__global__ void __launch_bounds__(512)
reduce_scatter_bf16_kernel(const __grid_constant__ PeerPtrs bufs, int rank, size_t start, size_t count, float* out_f32, float scale,
                           float* sumsq) {
  __shared__ float red[16];
  float ss = 0.f;
  const size_t nvec = count >> 3;  // 8 bf16 per 16 bytes
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int q = 0; q < N; ++q) {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bufs.p[(q + rank) % N]) + start) + i;
      uint4 v;
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                   : "l"(src)
                   : "memory");
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc[j] *= scale;
      ss += acc[j] * acc[j];
    }
    float4* dst = reinterpret_cast<float4*>(out_f32 + start) + 2 * i;
    dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  if (sumsq) {
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 16) {
      float t = red[threadIdx.x];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffu, t, o);
      if (threadIdx.x == 0) atomicAdd(sumsq, t);
    }
  }
}

struct AdamArgs2 {
  float lr, beta1, beta2, eps, wd, bc1, bc2, max_norm, grad_scale;
  int zero_grad, atan2_mode, n_ranks, push_master;
};

// AdamW on one shard [0, n) of a flat group (pointers already offset to the shard), pushing the bf16 compute copy
// (and optionally the fp32 master value) of every updated element to the same offset on all ranks.
__global__ void __launch_bounds__(256)
adamw_push_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                  const __grid_constant__ PeerPtrs shadows, const __grid_constant__ PeerPtrs masters, size_t n, const float* __restrict__ gnorm_sq, AdamArgs2 a) {
  float clip = 1.f;
  bool skip = false;
  if (gnorm_sq) {
    const float gn = sqrtf(*gnorm_sq) * a.grad_scale;
    if (!isfinite(gn)) skip = true;
    else if (a.max_norm > 0.f) clip = fminf(1.f, a.max_norm / (gn + 1e-6f));
  }
  const float gs = a.grad_scale * clip;
  const float inv_bc1 = 1.f / a.bc1, inv_sqrt_bc2 = rsqrtf(a.bc2);
  const size_t nvec = n >> 2;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    if (!skip) {
      const float4 gv = reinterpret_cast<float4*>(g)[i];
      float4 mv = reinterpret_cast<float4*>(m)[i];
      float4 vv = reinterpret_cast<float4*>(v)[i];
      float* pp = reinterpret_cast<float*>(&pv);
      const float* gp = reinterpret_cast<const float*>(&gv);
      float* mp = reinterpret_cast<float*>(&mv);
      float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = gp[j] * gs;
        mp[j] = mp[j] + (1.f - a.beta1) * (gj - mp[j]);
        vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gj * gj;
        float pj = pp[j] * (1.f - a.lr * a.wd);
        if (a.atan2_mode) pj -= a.lr * inv_bc1 * atan2f(mp[j], sqrtf(vp[j]) * inv_sqrt_bc2);
        else pj -= a.lr * inv_bc1 * mp[j] / (sqrtf(vp[j]) * inv_sqrt_bc2 + a.eps);
        pp[j] = pj;
      }
      reinterpret_cast<float4*>(p)[i] = pv;
      reinterpret_cast<float4*>(m)[i] = mv;
      reinterpret_cast<float4*>(v)[i] = vv;
    }
    if (a.zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    uint2 o;
    o.x = pack_bf16x2(pv.x, pv.y);
    o.y = pack_bf16x2(pv.z, pv.w);
    for (int q = 0; q < a.n_ranks; ++q) {
      reinterpret_cast<uint2*>(shadows.p[q])[i] = o;
      if (a.push_master) reinterpret_cast<float4*>(masters.p[q])[i] = pv;
    }
  }
}

}  // namespace b200

using namespace b200;

// ------------------------------------------------------------------------------------------------ IPC plumbing
B200_API int b200_ipc_alloc(long long bytes, void** ptr, void* handle64) {
  if (cudaMalloc(ptr, static_cast<size_t>(bytes)) != cudaSuccess) return -1;
  if (cudaMemset(*ptr, 0, static_cast<size_t>(bytes)) != cudaSuccess) return -2;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, *ptr) != cudaSuccess) return -3;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
B200_API int b200_ipc_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : -1;
}
B200_API int b200_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }
B200_API int b200_ipc_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }

static PeerPtrs make_ptrs(void* const* host_ptrs, int N, long long byte_offset = 0) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_RANKS; ++i)
    pp.p[i] = (i < N && host_ptrs && host_ptrs[i]) ? static_cast<char*>(host_ptrs[i]) + byte_offset : nullptr;
  return pp;
}

// flag_ptrs[q]: base of rank q's flag array (N uint32, zero-initialised).  partial_ptrs[q] (optional): one float
// on rank q that is summed into *total_out after the barrier.  timeout_ms bounds the wait.
B200_API int b200_barrier(void* const* flag_ptrs, int rank, int N, unsigned int epoch, int timeout_ms,
                          void* const* partial_ptrs, float* total_out, int* err, void* stream) {
  if (N > MAX_RANKS) return -1;
  barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      make_ptrs(flag_ptrs, N), rank, N, epoch, static_cast<unsigned long long>(timeout_ms) * 1000000ull,
      make_ptrs(partial_ptrs, N), partial_ptrs ? total_out : nullptr, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

#define DISPATCH_N(N_, CALL)                      \
  switch (N_) {                                   \
    case 2: { constexpr int NN = 2; CALL; break; } \
    case 3: { constexpr int NN = 3; CALL; break; } \
    case 4: { constexpr int NN = 4; CALL; break; } \
    case 5: { constexpr int NN = 5; CALL; break; } \
    case 6: { constexpr int NN = 6; CALL; break; } \
    case 7: { constexpr int NN = 7; CALL; break; } \
    case 8: { constexpr int NN = 8; CALL; break; } \
    default: return -1;                           \
  }

static inline int comm_grid(size_t nvec, int ctas) {
  size_t b = (nvec + 511) / 512;
  if (b < 1) b = 1;
  if (b > static_cast<size_t>(ctas)) b = ctas;
  return static_cast<int>(b);
}

// own[start:start+count) (fp32 elements) = sum over ranks; *sumsq += squared norm of the result.
B200_API int b200_reduce_scatter_f32(void* const* buf_ptrs, int rank, int N, long long start, long long count,
                                     float* sumsq, int ctas, void* stream) {
  if (count <= 0) return 0;
  if ((start & 3) || (count & 3)) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const PeerPtrs pp = make_ptrs(buf_ptrs, N);
  // ctas > 0: that many CTAs; bit 16 of `ctas` selects the variant without unrolling (for the communication sweep)
  const bool plain = ctas & 0x10000;
  ctas &= 0xffff;
  const int grid = comm_grid(count >> 2, ctas > 0 ? ctas : 296);
  if (plain) {
    DISPATCH_N(N, (reduce_scatter_kernel<NN, 1><<<grid, 512, 0, st>>>(pp, rank, start, count, sumsq)))
  } else {
    DISPATCH_N(N, (reduce_scatter_kernel<NN, (NN <= 4 ? 4 : 2)><<<grid, 512, 0, st>>>(pp, rank, start, count, sumsq)))
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// own[q * slice : (q+1) * slice) = buf_q[same range] for all q != rank; byte quantities, multiples of 16.
B200_API int b200_allgather_bytes(void* const* buf_ptrs, int rank, int N, long long slice_bytes, int ctas,
                                  void* stream) {
  if (slice_bytes <= 0) return 0;
  if (slice_bytes & 15) return -3;
  const size_t slice_vec = static_cast<size_t>(slice_bytes) >> 4;
  const int grid = comm_grid(slice_vec * N, ctas > 0 ? ctas : 296);
  allgather_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(make_ptrs(buf_ptrs, N), rank, N,
                                                                            slice_vec, slice_vec * N);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Push form of the all-gather: this rank's slice is stored into every peer.
B200_API int b200_allgather_push_bytes(void* const* buf_ptrs, int rank, int N, long long slice_bytes, int ctas,
                                       void* stream) {
  if (slice_bytes <= 0) return 0;
  if (slice_bytes & 15) return -3;
  const size_t slice_vec = static_cast<size_t>(slice_bytes) >> 4;
  const int grid = comm_grid(slice_vec, ctas > 0 ? ctas : 296);
  allgather_push_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(make_ptrs(buf_ptrs, N), rank, N,
                                                                                 slice_vec);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// out[0:count) = scale * sum over ranks of buf_q[0:count)  (fp32, one-shot; out must not be one of the bufs).
B200_API int b200_allreduce_oneshot_f32(void* const* buf_ptrs, int rank, int N, float* out, long long count,
                                        float scale, float* sumsq, int ctas, void* stream) {
  if (count <= 0) return 0;
  if (count & 3) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const PeerPtrs pp = make_ptrs(buf_ptrs, N);
  const int grid = comm_grid(count >> 2, ctas > 0 ? ctas : 296);
  DISPATCH_N(N, (allreduce_oneshot_kernel<NN><<<grid, 512, 0, st>>>(pp, rank, out, count, scale, sumsq)))
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// out_f32[start:start+count) = scale * sum over ranks of bf16 buf_q[start:start+count); count % 8 == 0.
B200_API int b200_reduce_scatter_bf16(void* const* buf_ptrs, int rank, int N, long long start, long long count,
                                      float* out_f32, float scale, float* sumsq, int ctas, void* stream) {
  if (count <= 0) return 0;
  if ((start & 7) || (count & 7)) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const PeerPtrs pp = make_ptrs(buf_ptrs, N);
  const int grid = comm_grid(count >> 3, ctas > 0 ? ctas : 296);
  DISPATCH_N(N, (reduce_scatter_bf16_kernel<NN><<<grid, 512, 0, st>>>(pp, rank, start, count, out_f32, scale, sumsq)))
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// AdamW on elements [start, start+count) of a flat group.  p, g: full local buffers (fp32); m, v: shard-sized state
// (element 0 corresponds to `start`); shadow_ptrs[q] / master_ptrs[q]: base of rank q's bf16 shadow / fp32 master
// buffer of this group (the update is pushed to all of them at the same offsets).
B200_API int b200_adamw_push(float* p, float* g, float* m, float* v, void* const* shadow_ptrs,
                             void* const* master_ptrs, int n_ranks, long long start, long long count,
                             const float* gnorm_sq, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                             float bc2, float max_norm, float grad_scale, int zero_grad, int atan2_mode,
                             void* stream) {
  if (count <= 0) return 0;
  if ((start & 3) || (count & 3)) return -3;
  AdamArgs2 a{lr, beta1, beta2, eps, wd, bc1, bc2, max_norm, grad_scale, zero_grad, atan2_mode, n_ranks,
              master_ptrs ? 1 : 0};
  size_t b = (static_cast<size_t>(count) / 4 + 255) / 256;
  if (b > 148 * 8) b = 148 * 8;
  if (b < 1) b = 1;
  adamw_push_kernel<<<static_cast<int>(b), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      p + start, g + start, m, v, make_ptrs(shadow_ptrs, n_ranks, start * 2), make_ptrs(master_ptrs, n_ranks, start * 4),
      static_cast<size_t>(count), gnorm_sq, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
