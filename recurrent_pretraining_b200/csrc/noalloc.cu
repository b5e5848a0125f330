// Allocation-free RMSNorm backward (see b200_noalloc.h for who needs it and the full contract).
//
// The per-CTA weight-gradient partials, which the regular entry point expects in a caller-allocated matrix, live
// in a file-scope __device__ array.  In host code that array's name is only a host-side stand-in, not a device
// address, so the set-up below asks the runtime for the real address once per device (cudaGetSymbolAddress, with
// that device current) and hands the pointer to the kernels.
#include "b200_noalloc.h"

#include <stdio.h>

#include "common.cuh"

namespace b200 {

static __device__ __align__(256) float g_noalloc_scratch[B200_NOALLOC_MAX_CTAS * B200_NOALLOC_MAX_E];

constexpr int NA_THREADS = 256;
constexpr int NA_MAXV = B200_NOALLOC_MAX_E / 8 / NA_THREADS;  // 8-element vectors per thread (4)

__device__ __forceinline__ float na_block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (NA_THREADS >> 5)) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

// Same arithmetic as rmsnorm_bwd_kernel; CTA b walks rows b, b + grid, ... and finally writes its dw partial to
// row b of `partial` (every row < grid and every column < E is written, so stale contents are never read).
__global__ void __launch_bounds__(NA_THREADS)
rmsnorm_bwd_noalloc_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                           const float* __restrict__ w, const float* __restrict__ rstd_in,
                           __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int M, int E) {
  __shared__ float red[32];
  const int nvec = E >> 3;
  float dwp[NA_MAXV][8];
#pragma unroll
  for (int i = 0; i < NA_MAXV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwp[i][j] = 0.f;
  for (size_t row = blockIdx.x; row < static_cast<size_t>(M); row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * E);
    const uint4* dr = reinterpret_cast<const uint4*>(dy + row * E);
    const float rstd = rstd_in[row];
    uint4 xq[NA_MAXV], dq[NA_MAXV];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NA_MAXV; ++i) {
      const int v = threadIdx.x + i * NA_THREADS;
      if (v < nvec) {
        xq[i] = xr[v];
        dq[i] = dr[v];
        const uint32_t qs[4] = {xq[i].x, xq[i].y, xq[i].z, xq[i].w}, ds[4] = {dq[i].x, dq[i].y, dq[i].z, dq[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 xf = unpack_bf16x2(qs[j]), df = unpack_bf16x2(ds[j]);
          const float h0 = xf.x * rstd, h1 = xf.y * rstd;
          dwp[i][2 * j] += df.x * bf2f(f2bf(h0));
          dwp[i][2 * j + 1] += df.y * bf2f(f2bf(h1));
          const float w0 = w ? w[v * 8 + 2 * j] : 1.f, w1 = w ? w[v * 8 + 2 * j + 1] : 1.f;
          dot += df.x * w0 * h0 + df.y * w1 * h1;
        }
      }
    }
    const float mean = na_block_sum(dot, red) / static_cast<float>(E);
#pragma unroll
    for (int i = 0; i < NA_MAXV; ++i) {
      const int v = threadIdx.x + i * NA_THREADS;
      if (v < nvec) {
        const uint32_t qs[4] = {xq[i].x, xq[i].y, xq[i].z, xq[i].w}, ds[4] = {dq[i].x, dq[i].y, dq[i].z, dq[i].w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 xf = unpack_bf16x2(qs[j]), df = unpack_bf16x2(ds[j]);
          const float w0 = w ? w[v * 8 + 2 * j] : 1.f, w1 = w ? w[v * 8 + 2 * j + 1] : 1.f;
          o[j] = pack_bf16x2(rstd * (df.x * w0 - xf.x * rstd * mean), rstd * (df.y * w1 - xf.y * rstd * mean));
        }
        reinterpret_cast<uint4*>(dx + row * E)[v] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  if (partial) {
#pragma unroll
    for (int i = 0; i < NA_MAXV; ++i) {
      const int v = threadIdx.x + i * NA_THREADS;
      if (v < nvec) {
        float* dst = partial + static_cast<size_t>(blockIdx.x) * E + v * 8;
        reinterpret_cast<float4*>(dst)[0] = make_float4(dwp[i][0], dwp[i][1], dwp[i][2], dwp[i][3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(dwp[i][4], dwp[i][5], dwp[i][6], dwp[i][7]);
      }
    }
  }
}

__global__ void noalloc_colsum_kernel(const float* __restrict__ in, float* __restrict__ out, int R, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int r = 0; r < R; ++r) s += in[static_cast<size_t>(r) * C + c];
  out[c] = s;
}

constexpr int NA_MAX_DEVICES = 64;
// Written without a lock: host threads that race on the first call of a device all store the same address.
static float* g_scratch_ptr[NA_MAX_DEVICES] = {nullptr};
static thread_local char g_last_error[256] = "";

static int fail(int code, const char* fmt, long a = 0, long b = 0) {
  snprintf(g_last_error, sizeof(g_last_error), fmt, a, b);
  return code;
}

// Device address of the scratch array for the current device; looked up on the first call per device.
static float* scratch_for_current_device(int* rc) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= NA_MAX_DEVICES) {
    *rc = fail(-3, "cannot identify the current CUDA device (error %ld, device %ld)", static_cast<long>(e), dev);
    return nullptr;
  }
  if (!g_scratch_ptr[dev]) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
      *rc = fail(-3, "cudaGetSymbolAddress failed for the scratch array (error %ld) on device %ld",
                 static_cast<long>(e), dev);
      return nullptr;
    }
    g_scratch_ptr[dev] = ptr;
  }
  return g_scratch_ptr[dev];
}

}  // namespace b200

using namespace b200;

B200_API const char* b200_noalloc_last_error(void) { return g_last_error; }

B200_API int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, void* dx,
                                      float* dw, int M, int E, void* stream) {
  g_last_error[0] = 0;
  if (E <= 0 || (E % 8) != 0 || E > B200_NOALLOC_MAX_E)
    return fail(-1, "row width E=%ld is not supported: it must be a multiple of 8 and at most %ld", E,
                B200_NOALLOC_MAX_E);
  if (M <= 0) return fail(-1, "row count M=%ld must be positive", M);
  // A bad pointer would fault on the device and take the caller's whole context with it: refuse it here instead.
  if (!dy || !x || !rstd || !dx) return fail(-1, "dy, x, rstd and dx must not be NULL");
  const uintptr_t vec = reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx);
  if (vec & 15) return fail(-1, "dy, x and dx must be 16-byte aligned (the kernel moves 8 bf16 values at a time)");
  const uintptr_t f32 = reinterpret_cast<uintptr_t>(rstd) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(dw);
  if (f32 & 3) return fail(-1, "w, rstd and dw must be 4-byte aligned");
  int rc = 0;
  float* scratch = scratch_for_current_device(&rc);
  if (!scratch) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int grid = M < B200_NOALLOC_MAX_CTAS ? M : B200_NOALLOC_MAX_CTAS;
  rmsnorm_bwd_noalloc_kernel<<<grid, NA_THREADS, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x), w, rstd,
      reinterpret_cast<__nv_bfloat16*>(dx), dw ? scratch : nullptr, M, E);
  if (dw) noalloc_colsum_kernel<<<(E + 127) / 128, 128, 0, st>>>(scratch, dw, grid, E);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(-2, "kernel launch failed (CUDA error %ld)", static_cast<long>(e));
  return 0;
}
