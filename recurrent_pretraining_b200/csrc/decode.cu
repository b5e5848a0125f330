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
template <bool F32_IN>
__global__ void rope_append_kernel(const void* __restrict__ qkv_in, const float* __restrict__ qk_bias,
                                   const float* __restrict__ cosT, const float* __restrict__ sinT,
                                   const int* __restrict__ pos, __nv_bfloat16* __restrict__ q_out,
                                   __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int B,
                                   int H, int Hkv, int D, int Lmax) {
  pdl_trigger();   // the successor may become resident now; it waits for this grid's completion before it reads
  pdl_wait();
  const int wq = H * D, wk = Hkv * D, wtot = wq + 2 * wk;
  const int vpr = wtot >> 3;
  const int gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= B * vpr) return;
  const int b = gid / vpr, c = (gid % vpr) << 3;
  const int p = pos[b];
  uint4 v;
  if constexpr (F32_IN) {  // the stream-K accumulator: round to bf16 as the plain GEMM store does, and re-arm it
    float4* src = reinterpret_cast<float4*>(const_cast<float*>(reinterpret_cast<const float*>(qkv_in)) +
                                            static_cast<size_t>(b) * wtot + c);
    const float4 f0 = src[0], f1 = src[1];
    src[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    src[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    v = make_uint4(pack_bf16x2(f0.x, f0.y), pack_bf16x2(f0.z, f0.w), pack_bf16x2(f1.x, f1.y), pack_bf16x2(f1.z, f1.w));
  } else {
    v = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(qkv_in) + static_cast<size_t>(b) * wtot)[c >> 3];
  }
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
  pdl_trigger();   // the successor may become resident now; it waits for this grid's completion before it reads
  pdl_wait();
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
  // U keys per group and trip: all 2 U loads are in flight together (the walk is latency-bound otherwise: one
  // dependent memory round trip per key), the U score reductions interleave, one softmax update covers the U keys
  constexpr int U = 4;
  for (int l = l0 + grp; l < l1; l += NG * U) {
    uint4 kk[U], vv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int lu = l + u * NG;
      kk[u] = vv[u] = make_uint4(0, 0, 0, 0);
      if (active && lu < l1) {
        kk[u] = __ldg(reinterpret_cast<const uint4*>(kb + lu * row));
        vv[u] = __ldg(reinterpret_cast<const uint4*>(vb + lu * row));
      }
    }
    float s[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t kw[4] = {kk[u].x, kk[u].y, kk[u].z, kk[u].w};
      s[u] = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16x2(kw[i]);
        s[u] += qv[2 * i] * f.x + qv[2 * i + 1] * f.y;
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
      for (int u = 0; u < U; ++u) s[u] += __shfl_xor_sync(gmask, s[u], o, 16);
    }
    float mn = m;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (l + u * NG >= l1) s[u] = -INFINITY;   // u = 0 is always a real key, so mn is finite below
      mn = fmaxf(mn, s[u]);
    }
    const float alpha = exp2f(m - mn);
    float pu[U], psum = 0.f;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      pu[u] = exp2f(s[u] - mn);
      psum += pu[u];
    }
    lsum = lsum * alpha + psum;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= alpha;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t vw[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16x2(vw[i]);
        acc[2 * i] += pu[u] * f.x;
        acc[2 * i + 1] += pu[u] * f.y;
      }
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
  pdl_trigger();   // the successor may become resident now; it waits for this grid's completion before it reads
  pdl_wait();
  constexpr int D = 32 * DPL;
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (idx >= total) return;
  // lane s holds split s's (max, sum) -- one parallel load instead of a serial walk (nsplit <= 32, checked by the host)
  const float2 ml = lane < nsplit ? *reinterpret_cast<const float2*>(part_ml + (static_cast<size_t>(idx) * nsplit + lane) * 2)
                                  : make_float2(-INFINITY, 0.f);
  float mm = ml.x;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
  const float a_mine = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - mm);
  const float ll = warp_sum(ml.y * a_mine);
  float o[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) o[i] = 0.f;
#pragma unroll 4
  for (int s = 0; s < nsplit; ++s) {
    const float a = __shfl_sync(0xffffffffu, a_mine, s);
    const size_t p = static_cast<size_t>(idx) * nsplit + s;
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
  pdl_trigger();   // the successor may become resident now; it waits for this grid's completion before it reads
  pdl_wait();
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
  pdl_trigger();   // the successor may become resident now; it waits for this grid's completion before it reads
  pdl_wait();
  const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i + 4 <= n) {
    const float4 v = *reinterpret_cast<float4*>(work + i);
    *reinterpret_cast<uint2*>(out + i) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    *reinterpret_cast<float4*>(work + i) = make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
    for (size_t k = i; k < n; ++k) { out[k] = f2bf(work[k]); work[k] = 0.f; }
  }
}

// y[t, i] = silu(g) * u with g = acc[t, i], u = acc[t, I + i] rounded to bf16 first (as the bf16 GEMM store would),
// acc = 0 afterwards: consumer of the stream-K gate-up projection.
__global__ void swiglu_acc_kernel(float* __restrict__ acc, __nv_bfloat16* __restrict__ y, size_t T, int I) {
  pdl_trigger();
  pdl_wait();
  const int vpr = I >> 2;
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= T * vpr) return;
  const size_t t = gid / vpr;
  const int c = static_cast<int>(gid % vpr) * 4;
  float4* gp = reinterpret_cast<float4*>(acc + t * 2 * I + c);
  float4* up = reinterpret_cast<float4*>(acc + t * 2 * I + I + c);
  const float4 g4 = *gp, u4 = *up;
  *gp = make_float4(0.f, 0.f, 0.f, 0.f);
  *up = make_float4(0.f, 0.f, 0.f, 0.f);
  const float g[4] = {bf2f(f2bf(g4.x)), bf2f(f2bf(g4.y)), bf2f(f2bf(g4.z)), bf2f(f2bf(g4.w))};
  const float u[4] = {bf2f(f2bf(u4.x)), bf2f(f2bf(u4.y)), bf2f(f2bf(u4.z)), bf2f(f2bf(u4.w))};
  float o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  *reinterpret_cast<uint2*>(y + t * I + c) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
}

// One CTA per row (decode batches have at most 64 rows):  s = bf16(a + x) with a in fp32 (then cleared) or bf16,
// y1 = norm(s) * w1 and, if w2 is given, y2 = norm(y1) * w2 -- the sandwich pair n2 -> n3 (or n4 -> next n1) in one
// launch.  Each norm rounds the normalised value to bf16 before the weight multiply, as the unfused kernels do.
template <bool A_F32>
__global__ void __launch_bounds__(256)
add_rmsnorm_pair_kernel(void* __restrict__ a, const __nv_bfloat16* __restrict__ x, const float* __restrict__ w1,
                        const float* __restrict__ w2, __nv_bfloat16* __restrict__ y1, __nv_bfloat16* __restrict__ y2,
                        int E, float eps) {
  pdl_trigger();   // the successor may become resident now; it waits for this grid's completion before it reads
  pdl_wait();
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

// Register-resident form of the kernel above for E % 8 == 0 and E <= 256 * 8 * NV: every thread owns NV vectors of
// eight channels, all global loads (a, x, both weights) are issued before the first reduction, and nothing is staged
// through y1 -- one memory round trip plus two block reductions instead of three dependent passes over the row.
template <bool A_F32, int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_pair_vec_kernel(void* __restrict__ a, const __nv_bfloat16* __restrict__ x, const float* __restrict__ w1,
                            const float* __restrict__ w2, __nv_bfloat16* __restrict__ y1, __nv_bfloat16* __restrict__ y2,
                            int E, float eps) {
  pdl_trigger();   // the successor may become resident now; it waits for this grid's completion before it reads
  pdl_wait();
  __shared__ float red[2][8];
  const size_t row = blockIdx.x;
  const int nvec = E >> 3;
  float v[NV][8], g1[NV][8], g2[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int idx = threadIdx.x + k * 256;
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[k][j] = 0.f; g1[k][j] = 1.f; g2[k][j] = 1.f; }
    if (idx < nvec) {
      const size_t off = row * E + static_cast<size_t>(idx) * 8;
      float av[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      uint4 xv = make_uint4(0u, 0u, 0u, 0u);
      if (x) xv = *reinterpret_cast<const uint4*>(x + off);
      if (a) {
        if constexpr (A_F32) {
          float4* ap = reinterpret_cast<float4*>(reinterpret_cast<float*>(a) + off);
          const float4 a0 = ap[0], a1 = ap[1];
          ap[0] = make_float4(0.f, 0.f, 0.f, 0.f);
          ap[1] = make_float4(0.f, 0.f, 0.f, 0.f);
          av[0] = a0.x; av[1] = a0.y; av[2] = a0.z; av[3] = a0.w;
          av[4] = a1.x; av[5] = a1.y; av[6] = a1.z; av[7] = a1.w;
        } else {
          const uint4 ab = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a) + off);
          const uint32_t aw[4] = {ab.x, ab.y, ab.z, ab.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 t = unpack_bf16x2(aw[j]); av[2 * j] = t.x; av[2 * j + 1] = t.y; }
        }
      }
      if (w1) {
        const float4 t0 = reinterpret_cast<const float4*>(w1)[2 * idx], t1 = reinterpret_cast<const float4*>(w1)[2 * idx + 1];
        g1[k][0] = t0.x; g1[k][1] = t0.y; g1[k][2] = t0.z; g1[k][3] = t0.w;
        g1[k][4] = t1.x; g1[k][5] = t1.y; g1[k][6] = t1.z; g1[k][7] = t1.w;
      }
      if (y2 && w2) {
        const float4 t0 = reinterpret_cast<const float4*>(w2)[2 * idx], t1 = reinterpret_cast<const float4*>(w2)[2 * idx + 1];
        g2[k][0] = t0.x; g2[k][1] = t0.y; g2[k][2] = t0.z; g2[k][3] = t0.w;
        g2[k][4] = t1.x; g2[k][5] = t1.y; g2[k][6] = t1.z; g2[k][7] = t1.w;
      }
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = unpack_bf16x2(xw[j]);
        const float s0 = bf2f(f2bf(av[2 * j] + t.x)), s1 = bf2f(f2bf(av[2 * j + 1] + t.y));
        v[k][2 * j] = s0;
        v[k][2 * j + 1] = s1;
        ss += s0 * s0 + s1 * s1;
      }
    }
  }
  auto block_total = [&](float t, int which) {
    t = warp_sum(t);
    if ((threadIdx.x & 31) == 0) red[which][threadIdx.x >> 5] = t;
    __syncthreads();
    float r = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) r += red[which][k];
    return r;
  };
  const float rstd1 = rsqrtf(block_total(ss, 0) / static_cast<float>(E) + eps);
  float ss2 = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int idx = threadIdx.x + k * 256;
    if (idx < nvec) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[k][j] = bf2f(f2bf(bf2f(f2bf(v[k][j] * rstd1)) * g1[k][j]));
        ss2 += v[k][j] * v[k][j];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = pack_bf16x2(v[k][2 * j], v[k][2 * j + 1]);
      *reinterpret_cast<uint4*>(y1 + row * E + static_cast<size_t>(idx) * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  if (!y2) return;
  const float rstd2 = rsqrtf(block_total(ss2, 1) / static_cast<float>(E) + eps);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int idx = threadIdx.x + k * 256;
    if (idx < nvec) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = pack_bf16x2(bf2f(f2bf(v[k][2 * j] * rstd2)) * g2[k][2 * j], bf2f(f2bf(v[k][2 * j + 1] * rstd2)) * g2[k][2 * j + 1]);
      *reinterpret_cast<uint4*>(y2 + row * E + static_cast<size_t>(idx) * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

}  // namespace b200

using namespace b200;

B200_API int b200_swiglu_acc(float* acc, void* y, long long T, int I, void* stream) {
  if (I % 4 || T <= 0) return -1;
  const size_t n = static_cast<size_t>(T) * (I / 4);
  launch_k(swiglu_acc_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
           acc, reinterpret_cast<__nv_bfloat16*>(y), static_cast<size_t>(T), I);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

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
  const int nv = (E % 8 == 0) ? (E / 8 + 255) / 256 : 0;
  const bool aligned = !((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y1) |
                          reinterpret_cast<uintptr_t>(y2) | reinterpret_cast<uintptr_t>(w1) | reinterpret_cast<uintptr_t>(w2)) & 15);
#define PAIR_VEC(NV)                                                                                                   \
  if (a_is_f32) launch_k(add_rmsnorm_pair_vec_kernel<true, NV>, dim3(rows), dim3(256), 0, st, a, xb, w1, w2, o1, o2, E, eps); \
  else launch_k(add_rmsnorm_pair_vec_kernel<false, NV>, dim3(rows), dim3(256), 0, st, a, xb, w1, w2, o1, o2, E, eps);
  if (aligned && nv == 1) { PAIR_VEC(1) }
  else if (aligned && nv == 2) { PAIR_VEC(2) }
  else if (aligned && nv == 3) { PAIR_VEC(3) }
  else if (aligned && nv == 4) { PAIR_VEC(4) }
  else if (a_is_f32) launch_k(add_rmsnorm_pair_kernel<true>, dim3(rows), dim3(256), 0, st, a, xb, w1, w2, o1, o2, E, eps);
  else launch_k(add_rmsnorm_pair_kernel<false>, dim3(rows), dim3(256), 0, st, a, xb, w1, w2, o1, o2, E, eps);
#undef PAIR_VEC
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// qkv_is_f32 != 0: qkv is the fp32 accumulator of a stream-K skinny GEMM (cleared after reading), else bf16.
B200_API int b200_rope_append(const void* qkv, const float* qk_bias, const float* cosT, const float* sinT,
                              const int* pos, void* q_out, void* k_cache, void* v_cache, int B, int H, int Hkv, int D,
                              int Lmax, void* stream, int qkv_is_f32) {
  if (D % 8) return -1;
  const int n = B * ((H + 2 * Hkv) * D / 8);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  __nv_bfloat16* qo = reinterpret_cast<__nv_bfloat16*>(q_out);
  __nv_bfloat16* kc = reinterpret_cast<__nv_bfloat16*>(k_cache);
  __nv_bfloat16* vc = reinterpret_cast<__nv_bfloat16*>(v_cache);
  if (qkv_is_f32)
    launch_k(rope_append_kernel<true>, dim3((n + 255) / 256), dim3(256), 0, st, qkv, qk_bias, cosT, sinT, pos, qo, kc, vc,
             B, H, Hkv, D, Lmax);
  else
    launch_k(rope_append_kernel<false>, dim3((n + 255) / 256), dim3(256), 0, st, qkv, qk_bias, cosT, sinT, pos, qo, kc, vc,
             B, H, Hkv, D, Lmax);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// scratch: part_o [B*H*splits*D] fp32, part_ml [B*H*splits*2] fp32 (caller-provided).
B200_API int b200_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* lens, void* out,
                                   float* part_o, float* part_ml, int B, int H, int Hkv, int D, int Lmax, int splits,
                                   float scale, void* stream) {
  if (D % 32 || D > 128 || splits < 1 || splits > 32 || ((Hkv * D) % 8)) return -1;
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
