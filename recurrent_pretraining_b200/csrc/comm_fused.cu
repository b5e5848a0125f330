// One-launch collectives on bf16 gradient buckets in symmetric memory: the cross-rank handshakes are inside the data
// kernel (no separate barrier launches), and the reduction is fused with the bf16 -> fp32 cast, a scale factor and the
// squared-norm partial; a second kernel does the clipped AdamW update of the reduced slice and pushes the new bf16
// parameters to every rank.
//
//   allreduce_bf16_kernel<N, PUSH = true>   "two-shot in one pass": every rank reduces its 1/N slice from all ranks and
//                                           stores the fp32 result into every rank's output buffer
//   allreduce_bf16_kernel<N, PUSH = false>  reduce-scatter: the result stays in the owner's output slice
//   allreduce_bf16_oneshot_kernel<N>        small buckets: every rank reduces the whole bucket itself (no stores to peers)
//   allgather_push_kernel2                  every rank stores its slice into all peers
//   adamw_slice_push_kernel                 waits for all ranks' norm partials, clips, updates its slice, pushes bf16
//
// Handshake protocol (per kernel): the first CTA publishes `epoch` in flag slot A of every rank ("my input is
// ready"); every CTA waits for all ranks' slot-A flags; after its last store each CTA fences and takes a ticket; the
// CTA with the last ticket publishes `epoch` in slot B ("I neither read your buffers nor write into them any more") and
// waits for all ranks' slot-B flags, so that when the kernel has finished on a rank, its input may be overwritten and
// its output is complete.  Waits are bounded; a time-out sets the status word, poisons the norm and the kernel returns.
// Peers are touched by plain loads and stores only.
#include "common.cuh"

namespace b200 {

constexpr int MAXR = 16;
struct PeerPtrsF {
  void* p[MAXR];
};

__device__ __forceinline__ void st_rel_sys(uint32_t* a, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acq_sys(const uint32_t* a) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_sys16(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

struct Handshake {
  PeerPtrsF slot_a, slot_b;   // per rank: base of the flag slot (MAXR x uint32), this rank writes entry [rank]
  int* ticket;                // device counter, zero between launches
  uint32_t epoch;
  unsigned long long timeout_ns;
  int* err;
};

// whole CTA; returns false on time-out
__device__ __forceinline__ bool wait_all(const uint32_t* mine, int N, uint32_t epoch, unsigned long long timeout_ns, int* err,
                                         int* s_flag) {
  if (threadIdx.x == 0) *s_flag = 0;
  __syncthreads();
  if (threadIdx.x < N) {
    const unsigned long long t0 = globaltimer_ns();
    while (static_cast<int32_t>(ld_acq_sys(mine + threadIdx.x) - epoch) < 0) {
      if (globaltimer_ns() - t0 > timeout_ns) {
        *s_flag = 1;
        if (err) atomicCAS(err, 0, ERR_WAIT_PEER_FLAG);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  return *s_flag == 0;
}

__device__ __forceinline__ bool hs_begin(const Handshake& h, int rank, int N, int* s_flag) {
  if (blockIdx.x == 0 && threadIdx.x < N) {
    __threadfence_system();
    st_rel_sys(reinterpret_cast<uint32_t*>(h.slot_a.p[threadIdx.x]) + rank, h.epoch);
  }
  return wait_all(reinterpret_cast<const uint32_t*>(h.slot_a.p[rank]), N, h.epoch, h.timeout_ns, h.err, s_flag);
}

__device__ __forceinline__ void hs_end(const Handshake& h, int rank, int N, int* s_flag) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_flag[1] = (atomicAdd(h.ticket, 1) == static_cast<int>(gridDim.x) - 1) ? 1 : 0;
  __syncthreads();
  if (!s_flag[1]) return;
  if (threadIdx.x < N) {
    __threadfence_system();
    st_rel_sys(reinterpret_cast<uint32_t*>(h.slot_b.p[threadIdx.x]) + rank, h.epoch);
  }
  wait_all(reinterpret_cast<const uint32_t*>(h.slot_b.p[rank]), N, h.epoch, h.timeout_ns, h.err, s_flag);
  if (threadIdx.x == 0) *h.ticket = 0;
}

__device__ __forceinline__ void block_sum_add(float v, float* red, float* dst) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0 && dst) atomicAdd(dst, t);
  }
  __syncthreads();
}

// out_q[lo .. hi) (fp32) = scale * sum over ranks of in_r[lo .. hi) (bf16) for this rank's slice [lo, hi) = [rank * per, ...);
// PUSH: stored into every rank's out, else only this rank's.  *sumsq += squared norm of the scaled result.
template <int N, bool PUSH>
__global__ void __launch_bounds__(512)
allreduce_bf16_kernel(const __grid_constant__ PeerPtrsF in, const __grid_constant__ PeerPtrsF out, int rank, long long per,
                      long long count, float scale, float* sumsq, const __grid_constant__ Handshake h) {
  __shared__ int s_flag[2];
  __shared__ float red[16];
  if (!hs_begin(h, rank, N, s_flag)) {
    if (sumsq && blockIdx.x == 0 && threadIdx.x == 0) *sumsq = __int_as_float(0x7fc00000);
    return;
  }
  long long lo = static_cast<long long>(rank) * per;
  if (lo > count) lo = count;
  long long hi = lo + per;
  if (hi > count) hi = count;
  const long long nvec = (hi - lo) >> 3;
  const uint4* src[N];
#pragma unroll
  for (int q = 0; q < N; ++q)
    src[q] = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(in.p[(q + rank) % N]) + lo);
  float ss = 0.f;
  constexpr int U = (N <= 4) ? 4 : 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += U * stride) {
    uint4 v[U][N];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < nvec) {
#pragma unroll
        for (int q = 0; q < N; ++q) v[u][q] = ld_sys16(src[q] + i + u * stride);
      }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long iv = i + u * stride;
      if (iv >= nvec) continue;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int q = 0; q < N; ++q) {
        const uint32_t w[4] = {v[u][q].x, v[u][q].y, v[u][q].z, v[u][q].w};
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
      const float4 a0 = make_float4(acc[0], acc[1], acc[2], acc[3]), a1 = make_float4(acc[4], acc[5], acc[6], acc[7]);
      if (PUSH) {
#pragma unroll
        for (int q = 0; q < N; ++q) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out.p[(q + rank) % N]) + lo) + 2 * iv;
          dst[0] = a0;
          dst[1] = a1;
        }
      } else {
        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out.p[rank]) + lo) + 2 * iv;
        dst[0] = a0;
        dst[1] = a1;
      }
    }
  }
  block_sum_add(ss, red, sumsq);
  hs_end(h, rank, N, s_flag);
}

// out (local fp32, whole bucket) = scale * sum over ranks of in_r (bf16); no stores to peers.
template <int N>
__global__ void __launch_bounds__(512)
allreduce_bf16_oneshot_kernel(const __grid_constant__ PeerPtrsF in, float* out, int rank, long long count, float scale,
                              float* sumsq, const __grid_constant__ Handshake h) {
  __shared__ int s_flag[2];
  __shared__ float red[16];
  if (!hs_begin(h, rank, N, s_flag)) {
    if (sumsq && blockIdx.x == 0 && threadIdx.x == 0) *sumsq = __int_as_float(0x7fc00000);
    return;
  }
  const long long nvec = count >> 3;
  float ss = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 v[N];
#pragma unroll
    for (int q = 0; q < N; ++q) v[q] = ld_sys16(reinterpret_cast<const uint4*>(in.p[(q + rank) % N]) + i);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int q = 0; q < N; ++q) {
      const uint32_t w[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
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
    float4* dst = reinterpret_cast<float4*>(out) + 2 * i;
    dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  block_sum_add(ss, red, sumsq);
  hs_end(h, rank, N, s_flag);
}

// Every rank stores its slice [rank * per_vec, ...) of 16-byte units into all peers' buffers.
__global__ void __launch_bounds__(512)
allgather_push_kernel2(const __grid_constant__ PeerPtrsF bufs, int rank, int N, long long per_vec, long long total_vec,
                       const __grid_constant__ Handshake h) {
  __shared__ int s_flag[2];
  if (!hs_begin(h, rank, N, s_flag)) return;
  long long lo = static_cast<long long>(rank) * per_vec;
  if (lo > total_vec) lo = total_vec;
  long long hi = lo + per_vec;
  if (hi > total_vec) hi = total_vec;
  const uint4* src = reinterpret_cast<const uint4*>(bufs.p[rank]) + lo;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < hi - lo;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
    for (int q = 1; q < N; ++q) reinterpret_cast<uint4*>(bufs.p[(rank + q) % N])[lo + i] = v;
  }
  hs_end(h, rank, N, s_flag);
}

struct SliceAdam {
  float lr, beta1, beta2, eps, decay, bc1, bc2, max_norm;
};

// AdamW on this rank's slice after a reduce-scatter: waits until every rank's squared-norm partial is final (slot A),
// sums them, clips, updates p / m / v (slice-local fp32 arrays of `n` elements, g the reduced fp32 gradient slice) and
// stores the new bf16 parameters at [lo, lo + n) of every rank's bf16 buffer.
__global__ void __launch_bounds__(256)
adamw_slice_push_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                        long long n, long long lo, const __grid_constant__ PeerPtrsF shadows,
                        const __grid_constant__ PeerPtrsF partials, int rank, int N, SliceAdam a, float* gnorm_out,
                        const __grid_constant__ Handshake h) {
  __shared__ int s_flag[2];
  __shared__ float s_clip;
  if (!hs_begin(h, rank, N, s_flag)) return;
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int q = 0; q < N; ++q) tot += *reinterpret_cast<const volatile float*>(partials.p[q]);
    const float gn = sqrtf(tot);
    if (gnorm_out && blockIdx.x == 0) *gnorm_out = gn;
    s_clip = !isfinite(gn) ? -1.f : (a.max_norm > 0.f ? fminf(1.f, a.max_norm / (gn + 1e-6f)) : 1.f);
  }
  __syncthreads();
  const float clip = s_clip;
  if (clip >= 0.f) {
    const float inv_sqrt_bc2 = rsqrtf(a.bc2), step = a.lr / a.bc1;
    const long long nvec = n >> 2;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float4 pv = reinterpret_cast<float4*>(p)[i];
      const float4 gv = reinterpret_cast<const float4*>(g)[i];
      float4 mv = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
      float* pp = reinterpret_cast<float*>(&pv);
      const float* gp = reinterpret_cast<const float*>(&gv);
      float* mp = reinterpret_cast<float*>(&mv);
      float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = gp[j] * clip;
        mp[j] += (1.f - a.beta1) * (gj - mp[j]);
        vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gj * gj;
        pp[j] = pp[j] * a.decay - step * mp[j] / (sqrtf(vp[j]) * inv_sqrt_bc2 + a.eps);
      }
      reinterpret_cast<float4*>(p)[i] = pv;
      reinterpret_cast<float4*>(m)[i] = mv;
      reinterpret_cast<float4*>(v)[i] = vv;
      uint2 o;
      o.x = pack_bf16x2(pv.x, pv.y);
      o.y = pack_bf16x2(pv.z, pv.w);
      for (int q = 0; q < N; ++q)
        reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(shadows.p[(q + rank) % N]) + lo)[i] = o;
    }
  }
  hs_end(h, rank, N, s_flag);
}

}  // namespace b200

using namespace b200;

static PeerPtrsF mkf(void* const* host_ptrs, int N, long long byte_offset = 0) {
  PeerPtrsF pp;
  for (int i = 0; i < MAXR; ++i)
    pp.p[i] = (i < N && host_ptrs && host_ptrs[i]) ? static_cast<char*>(host_ptrs[i]) + byte_offset : nullptr;
  return pp;
}
static Handshake mkh(void* const* slot_a, void* const* slot_b, int N, int* ticket, unsigned int epoch, int timeout_ms,
                     int* err) {
  Handshake h;
  h.slot_a = mkf(slot_a, N);
  h.slot_b = mkf(slot_b, N);
  h.ticket = ticket;
  h.epoch = epoch;
  h.timeout_ns = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  h.err = err;
  return h;
}
static inline int grid_of(long long nvec, int threads, int unroll, int ctas) {
  long long b = (nvec + static_cast<long long>(threads) * unroll - 1) / (static_cast<long long>(threads) * unroll);
  if (b < 1) b = 1;
  const int cap = ctas > 0 ? ctas : 296;
  return static_cast<int>(b > cap ? cap : b);
}

#define DISPATCH_NF(N_, CALL)                      \
  switch (N_) {                                    \
    case 2: { constexpr int NN = 2; CALL; break; } \
    case 3: { constexpr int NN = 3; CALL; break; } \
    case 4: { constexpr int NN = 4; CALL; break; } \
    case 5: { constexpr int NN = 5; CALL; break; } \
    case 6: { constexpr int NN = 6; CALL; break; } \
    case 7: { constexpr int NN = 7; CALL; break; } \
    case 8: { constexpr int NN = 8; CALL; break; } \
    default: return -1;                            \
  }

// mode 0: all-reduce (result in every rank's out), 1: reduce-scatter (result in the owner's out slice), 2: one-shot
// all-reduce (out is a LOCAL fp32 buffer passed as out_ptrs[rank]).  in: bf16 buckets; count elements (multiple of 8);
// per = elements per rank slice (multiple of 8).  slot_a / slot_b: flag slots (MAXR uint32 each) on every rank;
// ticket: zeroed int.
B200_API int b200_allreduce_bf16_fused(void* const* in_ptrs, void* const* out_ptrs, int rank, int N, long long per,
                                       long long count, float scale, float* sumsq, int mode, void* const* slot_a,
                                       void* const* slot_b, int* ticket, unsigned int epoch, int timeout_ms, int ctas,
                                       int* err, void* stream) {
  if (N < 2 || N > 8 || (count & 7) || (per & 7) || count <= 0) return -3;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const PeerPtrsF in = mkf(in_ptrs, N), out = mkf(out_ptrs, N);
  const Handshake h = mkh(slot_a, slot_b, N, ticket, epoch, timeout_ms, err);
  if (mode == 2) {
    const int grid = grid_of(count >> 3, 512, 1, ctas);
    DISPATCH_NF(N, (allreduce_bf16_oneshot_kernel<NN><<<grid, 512, 0, st>>>(in, reinterpret_cast<float*>(out_ptrs[rank]),
                                                                         rank, count, scale, sumsq, h)))
  } else {
    const int grid = grid_of(per >> 3, 512, 2, ctas);
    if (mode == 0) {
      DISPATCH_NF(N, (allreduce_bf16_kernel<NN, true><<<grid, 512, 0, st>>>(in, out, rank, per, count, scale, sumsq, h)))
    } else {
      DISPATCH_NF(N, (allreduce_bf16_kernel<NN, false><<<grid, 512, 0, st>>>(in, out, rank, per, count, scale, sumsq, h)))
    }
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Every rank's slice (per_bytes each, multiple of 16) of the symmetric buffers is stored into all peers.
B200_API int b200_allgather_push_fused(void* const* buf_ptrs, int rank, int N, long long per_bytes, long long total_bytes,
                                       void* const* slot_a, void* const* slot_b, int* ticket, unsigned int epoch,
                                       int timeout_ms, int ctas, int* err, void* stream) {
  if (N < 2 || N > MAXR || (per_bytes & 15) || (total_bytes & 15)) return -3;
  const Handshake h = mkh(slot_a, slot_b, N, ticket, epoch, timeout_ms, err);
  const int grid = grid_of(per_bytes >> 4, 512, 1, ctas);
  allgather_push_kernel2<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(mkf(buf_ptrs, N), rank, N,
                                                                                  per_bytes >> 4, total_bytes >> 4, h);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// AdamW on the slice reduced by a preceding reduce-scatter of this bucket (see adamw_slice_push_kernel).
// partial_ptrs[q]: rank q's squared-norm partial (one float in symmetric memory).
B200_API int b200_adamw_slice_push(float* p, const float* g, float* m, float* v, long long n, long long lo,
                                   void* const* shadow_ptrs, void* const* partial_ptrs, int rank, int N, float lr,
                                   float beta1, float beta2, float eps, float wd, float bc1, float bc2, float max_norm,
                                   float* gnorm_out, void* const* slot_a, void* const* slot_b, int* ticket,
                                   unsigned int epoch, int timeout_ms, int* err, void* stream) {
  if (N < 2 || N > MAXR || (n & 3) || (lo & 3) || n < 0) return -3;   // n == 0: handshakes only
  SliceAdam a{lr, beta1, beta2, eps, 1.f - lr * wd, bc1, bc2, max_norm};
  const Handshake h = mkh(slot_a, slot_b, N, ticket, epoch, timeout_ms, err);
  const int grid = grid_of(n >> 2, 256, 1, 148 * 4);
  adamw_slice_push_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      p, g, m, v, n, lo, mkf(shadow_ptrs, N), mkf(partial_ptrs, N), rank, N, a, gnorm_out, h);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
