// Fused optimizer kernels on flat fp32 buffers: squared-norm reduction and AdamW with the global-norm clip
// factor read from device memory, writing the updated fp32 master value, both moments, the bf16 compute
// copy of the parameter, and (optionally) zeroing the gradient for the next step -- one pass over memory.
#include "common.cuh"

namespace b200 {

__global__ void __launch_bounds__(256) sumsq_kernel(const float* __restrict__ g, size_t n, float* __restrict__ out) {
  __shared__ float red[8];
  float s = 0.f;
  const size_t nvec = n >> 2;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(g)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0) {
    for (size_t i = (nvec << 2) + threadIdx.x; i < n; i += blockDim.x) s += g[i] * g[i];
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffu, t, o);
    if (threadIdx.x == 0) atomicAdd(out, t);
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2;  // bc = 1 - beta^t
  float max_norm;                             // <= 0 disables clipping
  float grad_scale;                           // multiplies the stored gradient (1/world, 1/accum ...)
  int zero_grad;
  int atan2_mode;                             // ELLIS-style p -= step * atan2(m, sqrt(v / bc2))
};

// One element-wise pass.  gnorm_sq (device, may be null) holds sum(g^2) of the *unscaled* stored gradients;
// a non-finite norm skips the update (the step is a no-op, as in train.py:446-461 of the reference).
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             __nv_bfloat16* __restrict__ shadow, size_t n, const float* __restrict__ gnorm_sq, AdamArgs a) {
  float clip = 1.f;
  if (gnorm_sq) {
    const float gn = sqrtf(*gnorm_sq) * a.grad_scale;
    if (!isfinite(gn)) {
      if (a.zero_grad)
        for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
             i += static_cast<size_t>(gridDim.x) * blockDim.x)
          g[i] = 0.f;
      return;
    }
    if (a.max_norm > 0.f) clip = fminf(1.f, a.max_norm / (gn + 1e-6f));
  }
  const float gs = a.grad_scale * clip;
  const float inv_bc1 = 1.f / a.bc1, inv_sqrt_bc2 = rsqrtf(a.bc2);
  const size_t nvec = n >> 2;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    float4 gv = reinterpret_cast<float4*>(g)[i];
    float4 mv = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* pp = reinterpret_cast<float*>(&pv);
    float* gp = reinterpret_cast<float*>(&gv);
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
    if (a.zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (shadow) {
      uint2 o;
      o.x = pack_bf16x2(pp[0], pp[1]);
      o.y = pack_bf16x2(pp[2], pp[3]);
      reinterpret_cast<uint2*>(shadow)[i] = o;
    }
  }
  if (blockIdx.x == 0) {
    for (size_t i = (nvec << 2) + threadIdx.x; i < n; i += blockDim.x) {
      const float gj = g[i] * gs;
      const float mj = m[i] + (1.f - a.beta1) * (gj - m[i]);
      const float vj = a.beta2 * v[i] + (1.f - a.beta2) * gj * gj;
      float pj = p[i] * (1.f - a.lr * a.wd);
      if (a.atan2_mode) pj -= a.lr * inv_bc1 * atan2f(mj, sqrtf(vj) * inv_sqrt_bc2);
      else pj -= a.lr * inv_bc1 * mj / (sqrtf(vj) * inv_sqrt_bc2 + a.eps);
      p[i] = pj; m[i] = mj; v[i] = vj;
      if (a.zero_grad) g[i] = 0.f;
      if (shadow) shadow[i] = f2bf(pj);
    }
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n) {
  const size_t nvec = n >> 2;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(in)[i];
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    reinterpret_cast<uint2*>(out)[i] = o;
  }
  if (blockIdx.x == 0)
    for (size_t i = (nvec << 2) + threadIdx.x; i < n; i += blockDim.x) out[i] = f2bf(in[i]);
}

}  // namespace b200

using namespace b200;

static inline int grid_for(size_t n) {
  size_t b = (n / 4 + 255) / 256;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return static_cast<int>(b);
}

// *out += sum(g[i]^2); g must be 16-byte aligned.
B200_API int b200_sumsq(const float* g, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  sumsq_kernel<<<grid_for(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(g, static_cast<size_t>(n), out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_adamw(float* p, float* g, float* m, float* v, void* shadow, long long n, const float* gnorm_sq,
                        float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2, float max_norm,
                        float grad_scale, int zero_grad, int atan2_mode, void* stream) {
  if (n <= 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, max_norm, grad_scale, zero_grad, atan2_mode};
  adamw_kernel<<<grid_for(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      p, g, m, v, reinterpret_cast<__nv_bfloat16*>(shadow), static_cast<size_t>(n), gnorm_sq, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_cast_f32_bf16(const float* in, void* out, long long n, void* stream) {
  if (n <= 0) return 0;
  cast_f32_bf16_kernel<<<grid_for(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      in, reinterpret_cast<__nv_bfloat16*>(out), static_cast<size_t>(n));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
