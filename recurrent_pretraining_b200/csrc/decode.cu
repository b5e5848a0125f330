// Decode-side kernels of the native inference engine (all bandwidth-bound, bf16 data, fp32 math):
//   * rope_append   : q/k bias + RoPE for the single new position of every sequence, q written to a packed buffer,
//                     k and v appended in place to the per-recurrence-step cache slot [B, Lmax, Hkv, D]
//   * decode_attn   : one query row per (sequence, head) against the cached keys/values of one slot, keys split
//                     over `splits` CTAs with an online-softmax merge (flash-decoding); per-sequence lengths
//   * kl_exit       : log-softmax of the current logits, KL(prev || cur) against the previous recurrence step,
//                     threshold compare and first-exit bookkeeping, entirely on the device
#include "common.cuh"

namespace b200 {

// qkv: [B, (H + 2 Hkv) * D] for the new token of each sequence; pos[b]: its absolute position.
__global__ void rope_append_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ qk_bias,
                                   const float* __restrict__ cosT, const float* __restrict__ sinT,
                                   const int* __restrict__ pos, __nv_bfloat16* __restrict__ q_out,
                                   __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int B,
                                   int H, int Hkv, int D, int Lmax) {
  pdl_wait();
  pdl_trigger();
  const int wq = H * D, wk = Hkv * D, wtot = wq + 2 * wk;
  const int vpr = wtot >> 3;
  const int gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= B * vpr) return;
  const int b = gid / vpr, c = (gid % vpr) << 3;
  const int p = pos[b];
  uint4 v = reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(b) * wtot)[c >> 3];
  if (c < wq + wk) {
    const bool is_q = c < wq;
    const int cc = is_q ? c : c - wq;
    const int h = cc / D, d = cc % D;
    const float* cs = cosT + static_cast<size_t>(p) * (D >> 1) + (d >> 1);
    const float* sn = sinT + static_cast<size_t>(p) * (D >> 1) + (d >> 1);
    const float* bias = qk_bias ? qk_bias + (is_q ? 0 : H * D) + h * D + d : nullptr;
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16x2(w[j]);
      if (bias) f = unpack_bf16x2(pack_bf16x2(f.x + bias[2 * j], f.y + bias[2 * j + 1]));
      w[j] = pack_bf16x2(f.x * cs[j] - f.y * sn[j], f.y * cs[j] + f.x * sn[j]);
    }
    v = make_uint4(w[0], w[1], w[2], w[3]);
    if (is_q) {
      reinterpret_cast<uint4*>(q_out + static_cast<size_t>(b) * wq)[c >> 3] = v;
    } else {
      reinterpret_cast<uint4*>(k_cache + (static_cast<size_t>(b) * Lmax + p) * wk)[cc >> 3] = v;
    }
  } else {
    const int cc = c - wq - wk;
    reinterpret_cast<uint4*>(v_cache + (static_cast<size_t>(b) * Lmax + p) * wk)[cc >> 3] = v;
  }
}

// grid (splits, H, B), 128 threads = 8 groups of 16 lanes; group g walks keys l = begin + g, +8, ...; lane j of a
// group owns dims [8j, 8j+8) (one 16-byte load per key for K and for V).  Partial (m, l, o[D]) per split go to scratch
// and are merged by decode_attn_merge_kernel.  DPL = D / 32 (the merge kernel's layout).
template <int DPL>
__global__ void __launch_bounds__(128)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                   const __nv_bfloat16* __restrict__ vc, const int* __restrict__ lens, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int H, int Hkv, int Lmax, float scale_log2) {
  pdl_wait();
  pdl_trigger();
  constexpr int D = 32 * DPL;
  constexpr int NG = 8;  // key groups per CTA
  const int split = blockIdx.x, nsplit = gridDim.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (H / Hkv);
  const int grp = threadIdx.x >> 4, j = threadIdx.x & 15;
  const bool active = j * 8 < D;
  const int L = lens[b];
  const int per = (L + nsplit - 1) / nsplit;
  const int l0 = split * per, l1 = min(L, l0 + per);
  float qv[8], acc[8];
  const __nv_bfloat16* qp = q + (static_cast<size_t>(b) * H + h) * D;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    qv[i] = active ? bf2f(qp[j * 8 + i]) * scale_log2 : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, lsum = 0.f;
  const size_t row = static_cast<size_t>(Hkv) * D;
  const __nv_bfloat16* kb = kc + static_cast<size_t>(b) * Lmax * row + static_cast<size_t>(hk) * D + j * 8;
  const __nv_bfloat16* vb = vc + static_cast<size_t>(b) * Lmax * row + static_cast<size_t>(hk) * D + j * 8;
  const unsigned gmask = 0xFFFFu << (threadIdx.x & 16);  // the 16 lanes of this group inside the warp
  for (int l = l0 + grp; l < l1; l += NG) {
    float s = 0.f;
    uint4 vv = make_uint4(0, 0, 0, 0);
    if (active) {
      const uint4 kk = *reinterpret_cast<const uint4*>(kb + l * row);
      vv = *reinterpret_cast<const uint4*>(vb + l * row);
      const uint32_t kw[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16x2(kw[i]);
        s += qv[2 * i] * f.x + qv[2 * i + 1] * f.y;
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(gmask, s, o, 16);
    const float mn = fmaxf(m, s);
    const float alpha = exp2f(m - mn), p = exp2f(s - mn);
    lsum = lsum * alpha + p;
    const uint32_t vw[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack_bf16x2(vw[i]);
      acc[2 * i] = acc[2 * i] * alpha + p * f.x;
      acc[2 * i + 1] = acc[2 * i + 1] * alpha + p * f.y;
    }
    m = mn;
  }
  __shared__ float sm_m[NG], sm_l[NG], sm_o[NG][128];
  if (j == 0) { sm_m[grp] = m; sm_l[grp] = lsum; }
  if (active) {
#pragma unroll
    for (int i = 0; i < 8; ++i) sm_o[grp][j * 8 + i] = acc[i];
  }
  __syncthreads();
  if (threadIdx.x < D) {
    const int d = threadIdx.x;
    float mm = -INFINITY;
#pragma unroll
    for (int g = 0; g < NG; ++g) mm = fmaxf(mm, sm_m[g]);
    float ll = 0.f, o = 0.f;
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      const float a = (sm_m[g] == -INFINITY) ? 0.f : exp2f(sm_m[g] - mm);
      ll += sm_l[g] * a;
      o += sm_o[g][d] * a;
    }
    const size_t pidx = (static_cast<size_t>(b) * H + h) * nsplit + split;
    part_o[pidx * D + d] = o;
    if (d == 0) { part_ml[pidx * 2] = mm; part_ml[pidx * 2 + 1] = ll; }
  }
}

template <int DPL>
__global__ void decode_attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         __nv_bfloat16* __restrict__ out, int nsplit, int total /* B*H */) {
  pdl_wait();
  pdl_trigger();
  constexpr int D = 32 * DPL;
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (idx >= total) return;
  float mm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, part_ml[(static_cast<size_t>(idx) * nsplit + s) * 2]);
  float ll = 0.f, o[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) o[i] = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const size_t p = static_cast<size_t>(idx) * nsplit + s;
    const float ms = part_ml[p * 2];
    const float a = (ms == -INFINITY) ? 0.f : exp2f(ms - mm);
    ll += part_ml[p * 2 + 1] * a;
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] += part_o[p * D + lane + 32 * i] * a;
  }
  const float inv = ll > 0.f ? 1.f / ll : 0.f;
#pragma unroll
  for (int i = 0; i < DPL; ++i) out[static_cast<size_t>(idx) * D + lane + 32 * i] = f2bf(o[i] * inv);
}

// One CTA per sequence.  logits: [B, V] fp32 of the current recurrence step.  prev_logp: [B, V] fp32 (in/out).
// kl_out[b] = sum_v exp(prev) * (prev - cur).  exited[b] (in/out): set when kl < threshold and `armed` != 0;
// at a sequence's FIRST exit its step count and argmax token are recorded.  live_count: number of sequences
// that have not exited yet (host reads it every few steps instead of after every step).
__global__ void __launch_bounds__(512)
kl_exit_kernel(const float* __restrict__ logits, float* __restrict__ prev_logp, float* __restrict__ kl_out,
               int* __restrict__ exited, int* __restrict__ steps_taken, long long* __restrict__ token_out,
               int* __restrict__ live_count, int V, float threshold, int step, int armed) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[16];
  __shared__ int redi[16];
  __shared__ float s_val;
  const int b = blockIdx.x;
  const float* x = logits + static_cast<size_t>(b) * V;
  float* pl = prev_logp + static_cast<size_t>(b) * V;
  float m = -INFINITY;
  int am = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x)
    if (x[i] > m) { m = x[i]; am = i; }
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const int oi = __shfl_xor_sync(0xffffffffu, am, o);
    if (om > m || (om == m && oi < am)) { m = om; am = oi; }
  }
  if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = m; redi[threadIdx.x >> 5] = am; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w)
      if (red[w] > red[0] || (red[w] == red[0] && redi[w] < redi[0])) { red[0] = red[w]; redi[0] = redi[w]; }
    s_val = red[0];
  }
  __syncthreads();
  m = s_val;
  const int argmax = redi[0];
  __syncthreads();
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(x[i] - m);
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    s_val = m + __logf(t);
  }
  __syncthreads();
  const float lse = s_val;
  __syncthreads();
  float kl = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float cur = x[i] - lse, prev = pl[i];
    kl += __expf(prev) * (prev - cur);
    pl[i] = cur;
  }
  kl = warp_sum(kl);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = kl;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    kl_out[b] = t;
    if (!exited[b]) {
      token_out[b] = argmax;       // latest prediction; frozen once the sequence has exited
      steps_taken[b] = step + 1;
      if (armed && t < threshold) {
        exited[b] = 1;
        atomicSub(live_count, 1);
      }
    }
  }
}

// out = bf16(work); work = 0   (consumer of a split-K skinny GEMM that also re-arms its accumulator)
__global__ void cast_zero_kernel(float* __restrict__ work, __nv_bfloat16* __restrict__ out, size_t n) {
  pdl_wait();
  pdl_trigger();
  const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i + 4 <= n) {
    const float4 v = *reinterpret_cast<float4*>(work + i);
    *reinterpret_cast<uint2*>(out + i) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    *reinterpret_cast<float4*>(work + i) = make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
    for (size_t k = i; k < n; ++k) { out[k] = f2bf(work[k]); work[k] = 0.f; }
  }
}

// One CTA per row (decode batches have at most 64 rows):  s = bf16(a + x) with a in fp32 (then cleared) or bf16,
// y1 = norm(s) * w1 and, if w2 is given, y2 = norm(y1) * w2 -- the sandwich pair n2 -> n3 (or n4 -> next n1) in one
// launch.  Each norm rounds the normalised value to bf16 before the weight multiply, as the unfused kernels do.
template <bool A_F32>
__global__ void __launch_bounds__(256)
add_rmsnorm_pair_kernel(void* __restrict__ a, const __nv_bfloat16* __restrict__ x, const float* __restrict__ w1,
                        const float* __restrict__ w2, __nv_bfloat16* __restrict__ y1, __nv_bfloat16* __restrict__ y2,
                        int E, float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[8];
  __shared__ float s_tot;
  const size_t row = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x; i < E; i += 256) {
    float av = 0.f;
    if (a) {
      if constexpr (A_F32) {
        float* ap = reinterpret_cast<float*>(a) + row * E + i;
        av = *ap;
        *ap = 0.f;
      } else {
        av = bf2f(reinterpret_cast<const __nv_bfloat16*>(a)[row * E + i]);
      }
    }
    const float sv = bf2f(f2bf(av + (x ? bf2f(x[row * E + i]) : 0.f)));
    y1[row * E + i] = f2bf(sv);  // staged: overwritten with the normalised value below
    ss += sv * sv;
  }
  auto block_total = [&](float v) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int k = 0; k < 8; ++k) t += red[k];
      s_tot = t;
    }
    __syncthreads();
    const float r = s_tot;
    __syncthreads();
    return r;
  };
  const float rstd1 = rsqrtf(block_total(ss) / static_cast<float>(E) + eps);
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < E; i += 256) {
    const float sv = bf2f(y1[row * E + i]);
    const float o = bf2f(f2bf(bf2f(f2bf(sv * rstd1)) * (w1 ? w1[i] : 1.f)));
    y1[row * E + i] = f2bf(o);
    ss2 += o * o;
  }
  if (!y2) return;
  const float rstd2 = rsqrtf(block_total(ss2) / static_cast<float>(E) + eps);
  for (int i = threadIdx.x; i < E; i += 256) {
    const float o = bf2f(y1[row * E + i]);
    y2[row * E + i] = f2bf(bf2f(f2bf(o * rstd2)) * (w2 ? w2[i] : 1.f));
  }
}

}  // namespace b200

using namespace b200;

B200_API int b200_cast_zero(float* work, void* out, long long n, void* stream) {
  if (n <= 0) return 0;
  const size_t threads = (static_cast<size_t>(n) + 3) / 4;
  launch_k(cast_zero_kernel, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      work, reinterpret_cast<__nv_bfloat16*>(out), static_cast<size_t>(n));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// a: [rows, E] fp32 (a_is_f32, cleared after reading) or bf16 or null; y1 = n1(a + x); y2 = n2(y1) if y2 != null.
B200_API int b200_add_rmsnorm_pair(void* a, int a_is_f32, const void* x, const float* w1, const float* w2, void* y1,
                                   void* y2, int rows, int E, float eps, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* o1 = reinterpret_cast<__nv_bfloat16*>(y1);
  __nv_bfloat16* o2 = reinterpret_cast<__nv_bfloat16*>(y2);
  if (a_is_f32) launch_k(add_rmsnorm_pair_kernel<true>, dim3(rows), dim3(256), 0, st, a, xb, w1, w2, o1, o2, E, eps);
  else launch_k(add_rmsnorm_pair_kernel<false>, dim3(rows), dim3(256), 0, st, a, xb, w1, w2, o1, o2, E, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_rope_append(const void* qkv, const float* qk_bias, const float* cosT, const float* sinT,
                              const int* pos, void* q_out, void* k_cache, void* v_cache, int B, int H, int Hkv, int D,
                              int Lmax, void* stream) {
  if (D % 8) return -1;
  const int n = B * ((H + 2 * Hkv) * D / 8);
  launch_k(rope_append_kernel, dim3((n + 255) / 256), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      reinterpret_cast<const __nv_bfloat16*>(qkv), qk_bias, cosT, sinT, pos, reinterpret_cast<__nv_bfloat16*>(q_out),
      reinterpret_cast<__nv_bfloat16*>(k_cache), reinterpret_cast<__nv_bfloat16*>(v_cache), B, H, Hkv, D, Lmax);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// scratch: part_o [B*H*splits*D] fp32, part_ml [B*H*splits*2] fp32 (caller-provided).
B200_API int b200_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* lens, void* out,
                                   float* part_o, float* part_ml, int B, int H, int Hkv, int D, int Lmax, int splits,
                                   float scale, void* stream) {
  if (D % 32 || D > 128 || splits < 1 || ((Hkv * D) % 8)) return -1;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float sl2 = scale * 1.4426950408889634f;
  dim3 grid(splits, H, B);
  const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kb = reinterpret_cast<const __nv_bfloat16*>(k_cache);
  const __nv_bfloat16* vb = reinterpret_cast<const __nv_bfloat16*>(v_cache);
  __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(out);
  const int total = B * H;
#define RUN(DPL)                                                                                         \
  launch_k(decode_attn_kernel<DPL>, grid, dim3(128), 0, st, qb, kb, vb, lens, part_o, part_ml, H, Hkv, Lmax, sl2);  \
  launch_k(decode_attn_merge_kernel<DPL>, dim3((total + 3) / 4), dim3(128), 0, st, part_o, part_ml, ob, splits, total);
  switch (D / 32) {
    case 1: RUN(1) break;
    case 2: RUN(2) break;
    case 3: RUN(3) break;
    case 4: RUN(4) break;
    default: return -1;
  }
#undef RUN
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

B200_API int b200_kl_exit(const float* logits, float* prev_logp, float* kl_out, int* exited, int* steps_taken,
                          long long* token_out, int* live_count, int B, int V, float threshold, int step, int armed,
                          void* stream) {
  launch_k(kl_exit_kernel, dim3(B), dim3(512), 0, reinterpret_cast<cudaStream_t>(stream),logits, prev_logp, kl_out, exited, steps_taken,
                                                                      token_out, live_count, V, threshold, step, armed);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
