// Kernels of decoders whose attention layers keep keys and values in per-sequence rings: Dynamic-Tanh norms on an fp32
// residual stream, query/key preparation (whole-projection or per-head RMS norms, rotary positions with per-dimension
// frequencies), ring / kept-first-token caches, grouped-query attention under a position mask (chunks, or a sliding
// window that also keeps the first tokens of the sequence) for prompts and for single-token steps, and a
// mixture-of-experts feed-forward (sigmoid router with top-k choice, gated experts).
//
// Conventions (the same ragged-batch descriptor as seq_mixers.cu).  A step carries B sequences; sequence b brings
// n_b = seq_off[b+1]-seq_off[b] new tokens packed at rows seq_off[b].. of every activation matrix, has past[b] tokens
// already in its state, which lives in slot slots[b].  The token at packed row r of sequence b has position
// past[b] + r - seq_off[b].  Activations are `T` (float or bf16, `dtype` 0 / 1); softmax, norms, the router and the
// residual stream are fp32 in both.  Built WITHOUT fast-math: the fp32 mode is exact to rounding.
//
// Key/value rows.  A cache row is [G*D keys | G*V values] (C numbers) of one position.  Position p of a sequence
// lives at ring[slot][p % L]; positions below `nfirst` are also kept in first[slot][p] and never leave.  A prompt step
// reads its keys from an "ext" matrix: per sequence the rows [kept-first positions that are older than the contiguous
// part | cached positions cstart..past-1 | the step's own rows], ext_off[b] giving the first row, nsink[b] the number
// of rows of the first part and cstart[b] the position of the first row of the contiguous part.  A single-token step
// reads ring and `first` directly (its own row is written before).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

// dot product of a weight row with a vector staged in shared memory as fp32; the lanes of one warp share the row.
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const float* __restrict__ xs, int n, int lane);
template <>
__device__ __forceinline__ float warp_dot<float>(const float* __restrict__ w, const float* __restrict__ xs, int n, int lane) {
  float acc = 0.f;
  if ((n & 3) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
#pragma unroll 4
    for (int i = lane * 4; i < n; i += 128) {
      const float4 v = *reinterpret_cast<const float4*>(w + i);
      acc += v.x * xs[i] + v.y * xs[i + 1] + v.z * xs[i + 2] + v.w * xs[i + 3];
    }
  } else {
    for (int i = lane; i < n; i += 32) acc += w[i] * xs[i];
  }
  return warp_sum(acc);
}
template <>
__device__ __forceinline__ float warp_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ xs, int n,
                                                         int lane) {
  float acc = 0.f;
  if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
#pragma unroll 4
    for (int i = lane * 8; i < n; i += 256) {
      const uint4 raw = *reinterpret_cast<const uint4*>(w + i);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p[j]);
        acc += f.x * xs[i + 2 * j] + f.y * xs[i + 2 * j + 1];
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) acc += __bfloat162float(w[i]) * xs[i];
  }
  return warp_sum(acc);
}

// ------------------------------------------------------------------------------------------------------------------
// Embedding lookup with a constant factor into the fp32 stream: x[r] = table[ids[r]] * scale.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_scale_kernel(const T* __restrict__ table, const int64_t* __restrict__ ids, float scale, float* __restrict__ x,
                                   int n) {
  const long r = blockIdx.x;
  const T* src = table + ids[r] * (long)n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) x[r * n + i] = ldf(src + i) * scale;
}

// ------------------------------------------------------------------------------------------------------------------
// Dynamic Tanh norm, dyt(v) = tanh(alpha v) w + b (elementwise; no statistics), fused around the residual sum:
//   x[r] += dyt_post(y[r])      when y is given (y: rows of a sublayer's output, or — `pos` given — the weighted sum
//                               over `top` rows of a sorted expert output, y[pos[r,k]] * cw[r,k])
//   h[r]  = dyt_next(x[r])      when h is given
// x is the fp32 residual stream and is updated in place.
// ------------------------------------------------------------------------------------------------------------------
template <typename T, typename Ty>
__global__ void dyt_residual_kernel(float* __restrict__ x, const Ty* __restrict__ y, long ldy, const int* __restrict__ pos,
                                    const float* __restrict__ cw, int top, const T* __restrict__ pw, const T* __restrict__ pb,
                                    const T* __restrict__ palpha, const T* __restrict__ nw, const T* __restrict__ nb,
                                    const T* __restrict__ nalpha, T* __restrict__ h, long ldh, int n) {
  const long r = blockIdx.x;
  const float pa = y ? ldf(palpha) : 0.f, na = h ? ldf(nalpha) : 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = x[r * n + i];
    if (y) {
      float yv;
      if (pos) {
        yv = 0.f;
        for (int k = 0; k < top; ++k) yv += cw[r * top + k] * ldf(y + (long)pos[r * top + k] * ldy + i);
      } else {
        yv = ldf(y + r * ldy + i);
      }
      v += tanhf(pa * yv) * ldf(pw + i) + ldf(pb + i);
      x[r * n + i] = v;
    }
    if (h) stf(h + r * ldh + i, tanhf(na * v) * ldf(nw + i) + ldf(nb + i));
  }
}

// four consecutive channels per thread (n a multiple of 4, rows 16-byte aligned): 16-byte fp32 and 8-byte bf16 accesses
template <typename T> __device__ __forceinline__ float4 ld4(const T* p);
template <> __device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void st4(T* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T, typename Ty>
__global__ void dyt_residual_vec4_kernel(float* __restrict__ x, const Ty* __restrict__ y, long ldy, const int* __restrict__ pos,
                                         const float* __restrict__ cw, int top, const T* __restrict__ pw, const T* __restrict__ pb,
                                         const T* __restrict__ palpha, const T* __restrict__ nw, const T* __restrict__ nb,
                                         const T* __restrict__ nalpha, T* __restrict__ h, long ldh, int n) {
  const long r = blockIdx.x;
  const float pa = y ? ldf(palpha) : 0.f, na = h ? ldf(nalpha) : 0.f;
  for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(x + r * n + i);
    if (y) {
      float4 yv;
      if (pos) {
        yv = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < top; ++k) {
          const float w = cw[r * top + k];
          const float4 t = ld4<Ty>(y + (long)pos[r * top + k] * ldy + i);
          yv.x += w * t.x; yv.y += w * t.y; yv.z += w * t.z; yv.w += w * t.w;
        }
      } else {
        yv = ld4<Ty>(y + r * ldy + i);
      }
      const float4 w = ld4<T>(pw + i), b = ld4<T>(pb + i);
      v.x += tanhf(pa * yv.x) * w.x + b.x; v.y += tanhf(pa * yv.y) * w.y + b.y;
      v.z += tanhf(pa * yv.z) * w.z + b.z; v.w += tanhf(pa * yv.w) * w.w + b.w;
      *reinterpret_cast<float4*>(x + r * n + i) = v;
    }
    if (h) {
      const float4 w = ld4<T>(nw + i), b = ld4<T>(nb + i);
      st4<T>(h + r * ldh + i, make_float4(tanhf(na * v.x) * w.x + b.x, tanhf(na * v.y) * w.y + b.y, tanhf(na * v.z) * w.z + b.z,
                                          tanhf(na * v.w) * w.w + b.w));
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Elementwise activations between column slices: out = act(in), or — gated — out = act(in[:, :n]) * in[:, n:2n].
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float act_apply(float v, int act) {
  switch (act) {
    case 1: return 0.5f * v * (1.f + erff(v * 0.70710678118654752440f));                                   // gelu (erf)
    case 2: return v * sigmoidf_(v);                                                                          // silu
    case 3: return 0.5f * v * (1.f + tanhf(0.79788456080286535588f * (v + 0.044715f * v * v * v)));          // gelu (tanh)
    case 4: { const float r = fmaxf(v, 0.f); return r * r; }                                                 // relu squared
    default: return v;
  }
}
// gated pair (g, u) -> act(g) * u; act 5 is the clamped form  g' = min(g, limit), u' = clamp(u, -limit, limit),
// g' * sigmoid(1.702 g') * (u' + 1)
__device__ __forceinline__ float gated_apply(float g, float u, int act, float limit) {
  if (act == 5) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoidf_(1.702f * g) * (u + 1.f);
  }
  return act_apply(g, act) * u;
}
template <typename T>
__global__ void act_rows_kernel(const T* in, long ldi, T* out, long ldo, long rows, int n, int act, int gated, float limit) {   // in == out is allowed
  const long total = rows * n;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / n; const int c = (int)(i - r * n);
    float v = ldf(in + r * ldi + c);
    v = gated ? gated_apply(v, ldf(in + r * ldi + n + c), act, limit) : act_apply(v, act);
    stf(out + r * ldo + c, v);
  }
}

// bf16, 8 channels per thread with 16-byte accesses (n a multiple of 8, rows 16-byte aligned)
__global__ void act_rows_vec8_kernel(const __nv_bfloat16* in, long ldi, __nv_bfloat16* out, long ldo, long rows, int n, int act,
                                     int gated, float limit) {
  const int per = n / 8;
  const long total = rows * per;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / per; const int c = (int)(i - r * per) * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(in + r * ldi + c);
    uint4 b = make_uint4(0u, 0u, 0u, 0u);
    if (gated) b = *reinterpret_cast<const uint4*>(in + r * ldi + n + c);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 v = __bfloat1622float2(a2[j]);
      if (gated) { const float2 u = __bfloat1622float2(b2[j]); v.x = gated_apply(v.x, u.x, act, limit); v.y = gated_apply(v.y, u.y, act, limit); }
      else { v.x = act_apply(v.x, act); v.y = act_apply(v.y, act); }
      o2[j] = __floats2bfloat162_rn(v.x, v.y);
    }
    *reinterpret_cast<uint4*>(out + r * ldo + c) = o;
  }
}

__global__ void softcap_kernel(float* __restrict__ l, float cap, long total) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x)
    l[i] = cap * tanhf(l[i] / cap);
}

// ------------------------------------------------------------------------------------------------------------------
// Query / key preparation, in place, one block per token:
//   full_norm : q <- q / rms(q over all H*D) * qw, the same for k over all G*D (before rotation)
//   rotation  : the first `rot` channels of every head, channel i paired with i + rot/2, angle = position * freq[i];
//               cos and sin are multiplied by `mscale`
//   unit_norm : every head divided by its root mean square over D (after rotation, no weight)
// k may be absent (a layer that reads another layer's keys).
// ------------------------------------------------------------------------------------------------------------------
constexpr int QK_MAXD = 256;

template <typename T>
__global__ void __launch_bounds__(128)
qk_prepare_kernel(T* __restrict__ q, long ldq, T* __restrict__ k, long ldk, const T* __restrict__ qw, const T* __restrict__ kw,
                  const float* __restrict__ freq, float mscale, int rot, int H, int G, int D, float eps, int full_norm,
                  int unit_norm, const int* __restrict__ tok_seq, const int* __restrict__ seq_off, const int* __restrict__ past) {
  extern __shared__ float sm[];
  float* cs = sm; float* sn = sm + rot / 2; float* red = sm + rot;
  const long tok = blockIdx.x;
  const int b = tok_seq[tok];
  const int pos = past[b] + (int)(tok - seq_off[b]);
  const int half = rot / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * freq[i], &s, &c);
    cs[i] = c * mscale; sn[i] = s * mscale;
  }
  T* qr = q + tok * ldq;
  T* kr = k ? k + tok * ldk : nullptr;
  float rq = 1.f, rk = 1.f;
  if (full_norm) {
    // sums of squares over the whole projections; four channels per load where the rows allow it
    const bool v4 = (D & 3) == 0 && (ldq & 3) == 0 && (ldk & 3) == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0;
    float s = 0.f;
    if (v4) {
      for (int i = threadIdx.x * 4; i < H * D; i += blockDim.x * 4) { const float4 v = ld4<T>(qr + i); s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
    } else {
      for (int i = threadIdx.x; i < H * D; i += blockDim.x) { const float v = ldf(qr + i); s += v * v; }
    }
    rq = 1.f / sqrtf(block_sum(s, red) / (float)(H * D) + eps);
    if (kr) {
      s = 0.f;
      if (v4) {
        for (int i = threadIdx.x * 4; i < G * D; i += blockDim.x * 4) { const float4 v = ld4<T>(kr + i); s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
      } else {
        for (int i = threadIdx.x; i < G * D; i += blockDim.x) { const float v = ldf(kr + i); s += v * v; }
      }
      rk = 1.f / sqrtf(block_sum(s, red) / (float)(G * D) + eps);
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int heads = H + (kr ? G : 0);
  for (int hh = warp; hh < heads; hh += nw) {
    const bool isq = hh < H;
    T* p = isq ? qr + hh * D : kr + (hh - H) * D;
    const T* w = full_norm ? (isq ? qw + hh * D : kw + (hh - H) * D) : nullptr;
    const float sc = isq ? rq : rk;
    float ru[QK_MAXD / 64], rv[QK_MAXD / 64], rp[QK_MAXD / 32];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < QK_MAXD / 64; ++j) {
      const int i = lane + 32 * j;
      if (i < half) {
        float u = ldf(p + i) * sc, v = ldf(p + i + half) * sc;
        if (w) { u *= ldf(w + i); v *= ldf(w + i + half); }
        ru[j] = u * cs[i] - v * sn[i];
        rv[j] = v * cs[i] + u * sn[i];
        ss += ru[j] * ru[j] + rv[j] * rv[j];
      }
    }
#pragma unroll
    for (int j = 0; j < QK_MAXD / 32; ++j) {
      const int i = rot + lane + 32 * j;
      if (i < D) {
        float u = ldf(p + i) * sc;
        if (w) u *= ldf(w + i);
        rp[j] = u;
        ss += u * u;
      }
    }
    float un = 1.f;
    if (unit_norm) un = 1.f / sqrtf(warp_sum(ss) / (float)D + eps);
#pragma unroll
    for (int j = 0; j < QK_MAXD / 64; ++j) {
      const int i = lane + 32 * j;
      if (i < half) { stf(p + i, ru[j] * un); stf(p + i + half, rv[j] * un); }
    }
#pragma unroll
    for (int j = 0; j < QK_MAXD / 32; ++j) {
      const int i = rot + lane + 32 * j;
      if (i < D) stf(p + i, rp[j] * un);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Cache rows.  kv_write: the step's key rows (G*D) and value rows (G*V) go to ring[slot][pos % L] (only the last L of a
// sequence's new tokens) and, for pos < nfirst, to first[slot][pos].  kv_gather: builds the ext matrix of a prompt step.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void kv_write_kernel(T* __restrict__ ring, T* __restrict__ first, const T* __restrict__ knew, const T* __restrict__ vnew,
                                long ldn, const int* __restrict__ tok_seq, const int* __restrict__ seq_off,
                                const int* __restrict__ slots, const int* __restrict__ past, int KC, int VC, int L, int nfirst) {
  const long tok = blockIdx.x;
  const int b = tok_seq[tok];
  const int t = (int)(tok - seq_off[b]), n = seq_off[b + 1] - seq_off[b];
  const int pos = past[b] + t, C = KC + VC;
  const long slot = slots[b];
  if (n - t <= L) {
    T* dst = ring + (slot * L + pos % L) * C;
    for (int i = threadIdx.x; i < KC; i += blockDim.x) dst[i] = knew[tok * ldn + i];
    for (int i = threadIdx.x; i < VC; i += blockDim.x) dst[KC + i] = vnew[tok * ldn + i];
  }
  if (pos < nfirst) {
    T* dst = first + (slot * nfirst + pos) * C;
    for (int i = threadIdx.x; i < KC; i += blockDim.x) dst[i] = knew[tok * ldn + i];
    for (int i = threadIdx.x; i < VC; i += blockDim.x) dst[KC + i] = vnew[tok * ldn + i];
  }
}

template <typename T>
__global__ void kv_gather_kernel(const T* __restrict__ ring, const T* __restrict__ first, const T* __restrict__ knew,
                                 const T* __restrict__ vnew, long ldn, const int* __restrict__ ext_seq, const int* __restrict__ ext_off,
                                 const int* __restrict__ nsink, const int* __restrict__ cstart, const int* __restrict__ seq_off,
                                 const int* __restrict__ slots, const int* __restrict__ past, T* __restrict__ ext, int KC, int VC, int L,
                                 int nfirst) {
  const long r = blockIdx.x;
  const int b = ext_seq[r], C = KC + VC;
  const int rel = (int)(r - ext_off[b]), ns = nsink[b], cached = past[b] - cstart[b];
  const long slot = slots[b];
  T* dst = ext + r * C;
  if (rel < ns + cached) {
    const T* src = rel < ns ? first + (slot * nfirst + rel) * C : ring + (slot * L + (cstart[b] + rel - ns) % L) * C;
    for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = src[i];
  } else {
    const long tok = seq_off[b] + (rel - ns - cached);
    for (int i = threadIdx.x; i < KC; i += blockDim.x) dst[i] = knew[tok * ldn + i];
    for (int i = threadIdx.x; i < VC; i += blockDim.x) dst[KC + i] = vnew[tok * ldn + i];
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Grouped-query attention under a position mask.  The query at position i sees position j <= i when
//   chunk  > 0 : j >= floor(i / chunk) * chunk                                    (chunks counted from position 0)
//   window > 0 : j > i - window, or j < keep                                      (sliding window + kept first tokens)
// (neither: every j <= i).  Query head h reads key/value head h / (H/G).  One warp per (token, head): lanes take keys
// for the scores and value channels for the output; softmax in fp32, streamed 32 keys at a time.  The head's output is
// multiplied by sigmoid(gate[tok, h]) when a gate is given.  Keys come from the ext matrix (kbase/vbase with row stride
// ldkv) or, when `ring` is given, from ring / first (single-token steps).
//
// Options of every attention kernel of this file (AttnExtra): `softcap` > 0 passes the scaled scores through
// cap * tanh(score / cap); `sink` adds one entry of score 0 without a value to the softmax (its denominator grows by
// exp(0)); `gate_wide` reads one gate logit per output channel (gate[tok, h*V + c]) instead of one per head; the result
// is multiplied by `out_scale`.
// ------------------------------------------------------------------------------------------------------------------
struct AttnExtra { float softcap, out_scale; int sink, gate_wide; };
constexpr int ATT_MAXV = 8;    // value channels per lane: V <= 256

struct KvSource {
  const void* kbase; const void* vbase; long ldkv;            // ext mode
  const void* ring; const void* first; int L, nfirst, C, KC;  // ring mode
  const int* ext_off; const int* nsink; const int* cstart; const int* slots;
};

template <typename T>
__device__ __forceinline__ void kv_row(const KvSource& s, int b, int pos, int g, int D, int V, const T*& kp, const T*& vp) {
  if (s.ring) {
    const long slot = s.slots[b];
    const T* base = pos < s.nfirst ? (const T*)s.first + (slot * s.nfirst + pos) * s.C : (const T*)s.ring + (slot * s.L + pos % s.L) * s.C;
    kp = base + g * D; vp = base + s.KC + g * V;
  } else {
    const int cs = s.cstart[b];
    const long row = (long)s.ext_off[b] + (pos < cs ? pos : s.nsink[b] + pos - cs);
    kp = (const T*)s.kbase + row * s.ldkv + g * D; vp = (const T*)s.vbase + row * s.ldkv + g * V;
  }
}

template <typename T>
__global__ void masked_attention_kernel(const T* __restrict__ q, long ldq, KvSource src, const T* __restrict__ gate, long ldg,
                                        const int* __restrict__ tok_seq, const int* __restrict__ seq_off, const int* __restrict__ past,
                                        T* __restrict__ y, long ldy, long tokens, int H, int G, int D, int V, int window, int chunk,
                                        int keep, float scale, AttnExtra ex) {
  extern __shared__ float sm[];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long wid = (long)blockIdx.x * (blockDim.x >> 5) + wib;
  if (wid >= tokens * H) return;                 // no block-level sync below
  const long tok = wid / H; const int h = (int)(wid - tok * H);
  const int g = h / (H / G);
  const int b = tok_seq[tok];
  const int pi = past[b] + (int)(tok - seq_off[b]);
  int lo = 0;
  if (chunk > 0) lo = (pi / chunk) * chunk; else if (window > 0) lo = max(0, pi - window + 1);
  const int nA = (chunk > 0) ? 0 : min(keep, lo);
  const int total = nA + (pi - lo + 1);
  float* qs = sm + wib * D;
  for (int i = lane; i < D; i += 32) qs[i] = ldf(q + tok * ldq + h * D + i) * scale;
  __syncwarp();
  float m = -INFINITY, l = 0.f, acc[ATT_MAXV];
#pragma unroll
  for (int i = 0; i < ATT_MAXV; ++i) acc[i] = 0.f;
  for (int e = 0; e < total; e += 32) {
    const int mine = e + lane;
    float sc = -INFINITY;
    const T* kp = nullptr; const T* vp = nullptr;
    if (mine < total) {
      kv_row<T>(src, b, mine < nA ? mine : lo + mine - nA, g, D, V, kp, vp);
      float d = 0.f;
      for (int i = 0; i < D; ++i) d += qs[i] * ldf(kp + i);
      sc = ex.softcap > 0.f ? ex.softcap * tanhf(d / ex.softcap) : d;
    }
    const float mn = fmaxf(m, warp_max(sc));
    const float corr = expf(m - mn);             // m = -inf on the first block: exp(-inf) = 0
    const float p = mine < total ? expf(sc - mn) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ATT_MAXV; ++i) acc[i] *= corr;
    const int cnt = min(32, total - e);
    for (int kk = 0; kk < cnt; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const T* vr = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vp, kk);
#pragma unroll
      for (int i = 0; i < ATT_MAXV; ++i) { const int c = lane + 32 * i; if (c < V) acc[i] += pk * ldf(vr + c); }
    }
    m = mn;
  }
  if (ex.sink) l += expf(-m);                    // the entry of score 0 (m is finite: a query sees itself)
  const float gt = (gate && !ex.gate_wide) ? sigmoidf_(ldf(gate + tok * ldg + h)) : 1.f;
  const float inv = gt * ex.out_scale / l;
#pragma unroll
  for (int i = 0; i < ATT_MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < V) {
      const float gw = (gate && ex.gate_wide) ? sigmoidf_(ldf(gate + tok * ldg + h * V + c)) : 1.f;
      stf(y + tok * ldy + h * V + c, acc[i] * inv * gw);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// The same attention for prompts on the tensor cores (bf16 operands, fp32 accumulation and softmax): a block of 4 warps
// owns 64 consecutive queries of one (sequence, head) — 16 per warp, held as A fragments — and walks the ext rows its
// queries can see in tiles of 64 staged through shared memory: first the kept-first rows that lie before the tile's
// contiguous range, then the contiguous range.  S = Q Kᵀ with mma.m16n8k16, online softmax on the accumulator
// fragments, P re-packed as A fragments, O += P V with the V fragments fetched by ldmatrix.trans.  Query tiles are
// listed by the host (qt_seq / qt_start), so ragged batches cost no empty blocks.
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// cap * tanh(s / cap) for the tensor-core kernel: tanh(x) = 1 - 2 / (exp(2x) + 1), absolute error of a few 1e-7
__device__ __forceinline__ float soft_capped(float s, float cap, float inv_cap) {
  return cap * (1.f - __fdividef(2.f, __expf(2.f * s * inv_cap) + 1.f));
}
__device__ __forceinline__ int mask_floor(int p, int window, int chunk) {
  return chunk > 0 ? (p / chunk) * chunk : (window > 0 ? max(0, p - window + 1) : 0);
}

template <int D, int V>
__global__ void __launch_bounds__(128, 3)
masked_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, long ldq, const __nv_bfloat16* __restrict__ kbase,
                            const __nv_bfloat16* __restrict__ vbase, long ldkv, const int* __restrict__ ext_off,
                            const int* __restrict__ nsink, const int* __restrict__ cstart, const __nv_bfloat16* __restrict__ gate, long ldg,
                            const int* __restrict__ qt_seq, const int* __restrict__ qt_start, const int* __restrict__ seq_off,
                            const int* __restrict__ past, __nv_bfloat16* __restrict__ y, long ldy, int H, int G, int window, int chunk,
                            int keep, float scale, AttnExtra ex) {
  constexpr int KT = 64, KS = D + 8, VS = V + 8, BUF = KT * (KS + VS);
  extern __shared__ __align__(16) unsigned char mma_smem[];              // two buffers of [K tile | V tile]
  __nv_bfloat16* const tiles = reinterpret_cast<__nv_bfloat16*>(mma_smem);
  const int h = blockIdx.y, g = h / (H / G), b = qt_seq[blockIdx.x], t0 = qt_start[blockIdx.x];
  const int n = seq_off[b + 1] - seq_off[b], p0 = past[b];
  const long elo = ext_off[b];
  const int erows = ext_off[b + 1] - ext_off[b], ns = nsink[b], cs = cstart[b];
  const long tokbase = seq_off[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int r0 = t0 + warp * 16 + gid, r1 = r0 + 8;                    // this lane's two query rows
  const int pi0 = p0 + r0, pi1 = p0 + r1;                               // their positions
  const int lo0 = mask_floor(pi0, window, chunk), lo1 = mask_floor(pi1, window, chunk);
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int col = h * D + kk * 16 + tig * 2;
    qf[kk][0] = r0 < n ? *reinterpret_cast<const uint32_t*>(q + (tokbase + r0) * ldq + col) : 0u;
    qf[kk][1] = r1 < n ? *reinterpret_cast<const uint32_t*>(q + (tokbase + r1) * ldq + col) : 0u;
    qf[kk][2] = r0 < n ? *reinterpret_cast<const uint32_t*>(q + (tokbase + r0) * ldq + col + 8) : 0u;
    qf[kk][3] = r1 < n ? *reinterpret_cast<const uint32_t*>(q + (tokbase + r1) * ldq + col + 8) : 0u;
  }
  float o[V / 8][4];
#pragma unroll
  for (int j = 0; j < V / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;              // l: this lane's share of the row sums
  const int p_first = p0 + t0, p_last = p0 + min(t0 + 63, n - 1);
  const int lo_first = mask_floor(p_first, window, chunk);
  const int nA = chunk > 0 ? 0 : min(keep, lo_first);                   // kept-first rows before the contiguous range
  const int mrow0 = ns + lo_first - cs, mrow1 = ns + p_last - cs;       // contiguous range, as rows of this sequence
  const int pw0 = p0 + t0 + warp * 16, pw1 = pw0 + 15;                  // positions of this warp's queries
  const int low0 = mask_floor(pw0, window, chunk);
  const int tilesA = (nA + KT - 1) / KT, tilesB = (mrow1 - mrow0) / KT + 1, ntiles = tilesA + tilesB;
  // tile `it` goes to buffer it & 1 by cp.async (rows at or beyond the tile's limit are zero-filled: source size 0); the
  // copy of tile it + 1 is in flight while tile it is multiplied
  auto prefetch = [&](int it) {
    const bool pa = it < tilesA;
    const int k0 = pa ? it * KT : mrow0 + (it - tilesA) * KT, rlim = pa ? nA : erows;
    __nv_bfloat16* kd = tiles + (it & 1) * BUF;
    __nv_bfloat16* vd = kd + KT * KS;
    for (int c = threadIdx.x; c < KT * (D / 8); c += 128) {
      const int row = c / (D / 8), ch = c - row * (D / 8);
      const bool ok = k0 + row < rlim;
      const __nv_bfloat16* src = kbase + (elo + (ok ? k0 + row : 0)) * ldkv + g * D + ch * 8;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(kd + row * KS + ch * 8)),
                   "l"(src), "r"(ok ? 16 : 0));
    }
    for (int c = threadIdx.x; c < KT * (V / 8); c += 128) {
      const int row = c / (V / 8), ch = c - row * (V / 8);
      const bool ok = k0 + row < rlim;
      const __nv_bfloat16* src = vbase + (elo + (ok ? k0 + row : 0)) * ldkv + g * V + ch * 8;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(vd + row * VS + ch * 8)),
                   "l"(src), "r"(ok ? 16 : 0));
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  prefetch(0);
  for (int it = 0; it < ntiles; ++it) {
    const bool phaseA = it < tilesA;
    const int k0 = phaseA ? it * KT : mrow0 + (it - tilesA) * KT;       // first row of the tile
    const int rlim = phaseA ? nA : erows;                                // rows of the tile at or beyond it do not count
    if (it + 1 < ntiles) {
      prefetch(it + 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();                                                      // every thread's part of tile `it` has landed
    const __nv_bfloat16* Ks = tiles + (it & 1) * BUF;
    const __nv_bfloat16* Vs = Ks + KT * KS;
    bool skip = false;
    if (!phaseA) {                                                        // nothing in this tile for the warp's 16 queries?
      const int kp0 = cs + k0 - ns, kp1 = kp0 + KT - 1;                  // positions of the tile's first and last row
      skip = kp0 > pw1 || (kp1 < low0 && kp0 >= keep);
    }
    if (!skip) {
    float sacc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) { sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f; }
    // B fragments of two key blocks (j, j + 1) per ldmatrix.x4: lanes 0-7 / 8-15 address the rows of block j at channels
    // kk*16 / kk*16 + 8, lanes 16-23 / 24-31 the same of block j + 1
    const uint32_t krow = (uint32_t)__cvta_generic_to_shared(&Ks[((lane >> 4) * 8 + (lane & 7)) * KS + ((lane >> 3) & 1) * 8]);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(krow + (j * 8 * KS + kk * 16) * 2));
        mma_bf16(sacc[j], qf[kk], b0, b1);
        mma_bf16(sacc[j + 1], qf[kk], b2, b3);
      }
    }
    const bool capped = ex.softcap > 0.f;
    const float inv_cap = capped ? 1.f / ex.softcap : 0.f;
    float mx0 = -INFINITY, mx1 = -INFINITY;
    // a tile that every query of the warp sees completely needs no mask (warp-uniform)
    const bool whole = phaseA ? (k0 + KT <= rlim)
                              : (k0 + KT <= rlim && cs + k0 - ns + KT - 1 <= pw0 && cs + k0 - ns >= mask_floor(pw1, window, chunk));
    if (whole) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float sv = sacc[j][c] * scale;
          if (capped) sv = soft_capped(sv, ex.softcap, inv_cap);
          sacc[j][c] = sv;
          if (c < 2) mx0 = fmaxf(mx0, sv); else mx1 = fmaxf(mx1, sv);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int row = k0 + j * 8 + tig * 2 + (c & 1);
          const int pj = row < ns ? row : cs + row - ns;
          const int pi = c < 2 ? pi0 : pi1, lo = c < 2 ? lo0 : lo1;
          const bool valid = row < rlim && pj <= pi && (phaseA || pj >= lo || pj < keep);
          float sv = sacc[j][c] * scale;
          if (capped) sv = soft_capped(sv, ex.softcap, inv_cap);
          if (!valid) sv = -INFINITY;
          sacc[j][c] = sv;
          if (c < 2) mx0 = fmaxf(mx0, sv); else mx1 = fmaxf(mx1, sv);
        }
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float c0 = mn0 == -INFINITY ? 1.f : __expf(m0 - mn0), c1 = mn1 == -INFINITY ? 1.f : __expf(m1 - mn1);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float sv = sacc[j][c];
        const float pv = sv == -INFINITY ? 0.f : __expf(sv - (c < 2 ? mn0 : mn1));
        sacc[j][c] = pv;
        if (c < 2) s0 += pv; else s1 += pv;
      }
    }
    l0 = l0 * c0 + s0; l1 = l1 * c1 + s1; m0 = mn0; m1 = mn1;
    if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {              // a row maximum moved: rescale (multiplying by 1 is exact, so skipping is too)
#pragma unroll
      for (int j = 0; j < V / 8; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
    }
#pragma unroll
    for (int k2 = 0; k2 < 4; ++k2) {
      uint32_t a[4];
      a[0] = pack_bf16(sacc[2 * k2][0], sacc[2 * k2][1]); a[1] = pack_bf16(sacc[2 * k2][2], sacc[2 * k2][3]);
      a[2] = pack_bf16(sacc[2 * k2 + 1][0], sacc[2 * k2 + 1][1]); a[3] = pack_bf16(sacc[2 * k2 + 1][2], sacc[2 * k2 + 1][3]);
      // V fragments of two channel blocks (j, j + 1) per ldmatrix.x4.trans: lanes 0-15 address the 16 key rows at channels
      // j*8, lanes 16-31 the same rows at channels (j + 1)*8
      const uint32_t vrow = (uint32_t)__cvta_generic_to_shared(&Vs[(k2 * 16 + (lane & 15)) * VS + (lane >> 4) * 8]);
#pragma unroll
      for (int j = 0; j < V / 8; j += 2) {
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(vrow + j * 16));
        mma_bf16(o[j], a, b0, b1);
        mma_bf16(o[j + 1], a, b2, b3);
      }
    }
      }                                                                   // (!skip)
    __syncthreads();                                                      // all warps are done with this buffer before tile it + 2 overwrites it
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (ex.sink) { l0 += __expf(-m0); l1 += __expf(-m1); }                // the entry of score 0 (rows beyond n: 0 / inf = 0, never stored)
  const bool narrow = gate && !ex.gate_wide, wide = gate && ex.gate_wide;
  const float g0 = (narrow && r0 < n) ? sigmoidf_(__bfloat162float(gate[(tokbase + r0) * ldg + h])) : 1.f;
  const float g1 = (narrow && r1 < n) ? sigmoidf_(__bfloat162float(gate[(tokbase + r1) * ldg + h])) : 1.f;
  const float i0 = g0 * ex.out_scale / l0, i1 = g1 * ex.out_scale / l1;
#pragma unroll
  for (int j = 0; j < V / 8; ++j) {
    const int col = h * V + j * 8 + tig * 2;
    float a0 = o[j][0] * i0, a1 = o[j][1] * i0, b0 = o[j][2] * i1, b1 = o[j][3] * i1;
    if (wide) {
      if (r0 < n) {
        const __nv_bfloat162 gg = *reinterpret_cast<const __nv_bfloat162*>(gate + (tokbase + r0) * ldg + col);
        a0 *= sigmoidf_(__low2float(gg)); a1 *= sigmoidf_(__high2float(gg));
      }
      if (r1 < n) {
        const __nv_bfloat162 gg = *reinterpret_cast<const __nv_bfloat162*>(gate + (tokbase + r1) * ldg + col);
        b0 *= sigmoidf_(__low2float(gg)); b1 *= sigmoidf_(__high2float(gg));
      }
    }
    if (r0 < n) *reinterpret_cast<uint32_t*>(y + (tokbase + r0) * ldy + col) = pack_bf16(a0, a1);
    if (r1 < n) *reinterpret_cast<uint32_t*>(y + (tokbase + r1) * ldy + col) = pack_bf16(b0, b1);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Single-token steps, grouped: a block owns one (sequence, key/value head) and one of `splits` parts of the visible
// positions, so a key / value row is read once for all R = H/G query heads that share it.  Each of the 4 warps takes
// groups of 32 positions (a lane computes the R scores of its position, then the lanes share the value channels);
// the warps' partial softmaxes are merged in shared memory and written as (max, sum, weighted values) per part; a
// second kernel merges the parts, applies the head gate and writes the output.
// ------------------------------------------------------------------------------------------------------------------
constexpr int DEC_MAXR = 8, DEC_MAXVL = 4;     // query heads per key head; value channels per lane (V <= 128)

template <typename T> struct Vec8 {};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 t = __bfloat1622float2(h2[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
  }
};

template <typename T>
__global__ void __launch_bounds__(128)
ring_decode_kernel(const T* __restrict__ q, long ldq, const T* __restrict__ ring, const T* __restrict__ first, int L, int nfirst,
                   const int* __restrict__ slots, const int* __restrict__ past, float* __restrict__ part, int H, int G, int D, int V,
                   int window, int chunk, int keep, float scale, int splits, int vec, float softcap) {
  extern __shared__ float sm[];
  const int b = blockIdx.x, g = blockIdx.y, sp = blockIdx.z;
  const int R = H / G, C = G * (D + V), KC = G * D;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = sm;                                   // [R][D] scaled queries
  float* red = sm + R * D;                          // [4 warps][R][V + 2]
  for (int i = threadIdx.x; i < R * D; i += blockDim.x) qs[i] = ldf(q + (long)b * ldq + (long)g * R * D + i) * scale;
  __syncthreads();
  const int pi = past[b];
  const long slot = slots[b];
  const int lo = mask_floor(pi, window, chunk);
  const int nA = chunk > 0 ? 0 : min(keep, lo);
  const int total = nA + (pi - lo + 1);
  const int per = ((total + splits - 1) / splits + 31) / 32 * 32;
  const int v0 = sp * per, v1 = min(total, v0 + per);
  float m[DEC_MAXR], l[DEC_MAXR], acc[DEC_MAXR][DEC_MAXVL];
#pragma unroll
  for (int r = 0; r < DEC_MAXR; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < DEC_MAXVL; ++c) acc[r][c] = 0.f;
  }
  for (int e = v0 + warp * 32; e < v1; e += 128) {
    const int mine = e + lane;
    float sc[DEC_MAXR];
#pragma unroll
    for (int r = 0; r < DEC_MAXR; ++r) sc[r] = -INFINITY;
    const T* vp = nullptr;
    if (mine < v1) {
      const int pj = mine < nA ? mine : lo + mine - nA;
      const T* base = pj < nfirst ? first + (slot * nfirst + pj) * C : ring + (slot * L + pj % L) * C;
      const T* kp = base + g * D;
      vp = base + KC + g * V;
#pragma unroll
      for (int r = 0; r < DEC_MAXR; ++r) sc[r] = 0.f;
      if (vec) {
        for (int i = 0; i < D; i += 8) {
          float kf[8];
          Vec8<T>::load(kp + i, kf);
#pragma unroll
          for (int r = 0; r < DEC_MAXR; ++r) {
            if (r < R) {
              const float* qr = qs + r * D + i;
#pragma unroll
              for (int j = 0; j < 8; ++j) sc[r] += qr[j] * kf[j];
            }
          }
        }
      } else {
        for (int i = 0; i < D; ++i) {
          const float kv = ldf(kp + i);
#pragma unroll
          for (int r = 0; r < DEC_MAXR; ++r) if (r < R) sc[r] += qs[r * D + i] * kv;
        }
      }
#pragma unroll
      for (int r = 0; r < DEC_MAXR; ++r) {
        if (r >= R) sc[r] = -INFINITY;
        else if (softcap > 0.f) sc[r] = softcap * tanhf(sc[r] / softcap);
      }
    }
    float p[DEC_MAXR];
#pragma unroll
    for (int r = 0; r < DEC_MAXR; ++r) {
      p[r] = 0.f;
      if (r < R) {
        const float mn = fmaxf(m[r], warp_max(sc[r]));
        const float corr = expf(m[r] - mn);
        p[r] = mine < v1 ? expf(sc[r] - mn) : 0.f;
        l[r] = l[r] * corr + warp_sum(p[r]);
#pragma unroll
        for (int c = 0; c < DEC_MAXVL; ++c) acc[r][c] *= corr;
        m[r] = mn;
      }
    }
    const int cnt = min(32, v1 - e);
    for (int kk = 0; kk < cnt; ++kk) {
      const T* vr = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vp, kk);
      float vv[DEC_MAXVL];
#pragma unroll
      for (int c = 0; c < DEC_MAXVL; ++c) { const int ch = lane + 32 * c; vv[c] = ch < V ? ldf(vr + ch) : 0.f; }
#pragma unroll
      for (int r = 0; r < DEC_MAXR; ++r) {
        if (r < R) {
          const float pk = __shfl_sync(0xffffffffu, p[r], kk);
#pragma unroll
          for (int c = 0; c < DEC_MAXVL; ++c) acc[r][c] += pk * vv[c];
        }
      }
    }
  }
  // merge the 4 warps
  const int W = V + 2;
#pragma unroll
  for (int r = 0; r < DEC_MAXR; ++r) {
    if (r < R) {
      float* dst = red + ((long)warp * R + r) * W;
      if (lane == 0) { dst[0] = m[r]; dst[1] = l[r]; }
#pragma unroll
      for (int c = 0; c < DEC_MAXVL; ++c) { const int ch = lane + 32 * c; if (ch < V) dst[2 + ch] = acc[r][c]; }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < R * V; i += blockDim.x) {
    const int r = i / V, ch = i - r * V;
    float mm = -INFINITY;
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[((long)w * R + r) * W]);
    float ll = 0.f, a = 0.f;
    for (int w = 0; w < 4; ++w) {
      const float* src = red + ((long)w * R + r) * W;
      const float f = src[0] == -INFINITY ? 0.f : expf(src[0] - mm);
      ll += src[1] * f; a += src[2 + ch] * f;
    }
    float* dst = part + (((long)b * H + g * R + r) * splits + sp) * W;
    if (ch == 0) { dst[0] = mm; dst[1] = ll; }
    dst[2 + ch] = a;
  }
}

template <typename T>
__global__ void ring_decode_merge_kernel(const float* __restrict__ part, const T* __restrict__ gate, long ldg, T* __restrict__ y, long ldy,
                                         int H, int V, int splits, AttnExtra ex) {
  const int b = blockIdx.x, h = blockIdx.y, W = V + 2;
  const float* src = part + ((long)b * H + h) * splits * W;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, src[s * W]);
  float ll = 0.f;
  for (int s = 0; s < splits; ++s) ll += src[s * W] == -INFINITY ? 0.f : src[s * W + 1] * expf(src[s * W] - mm);
  if (ex.sink) ll += expf(-mm);                  // the entry of score 0
  const float gt = (gate && !ex.gate_wide) ? sigmoidf_(ldf(gate + (long)b * ldg + h)) : 1.f;
  for (int ch = threadIdx.x; ch < V; ch += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s) a += src[s * W] == -INFINITY ? 0.f : src[s * W + 2 + ch] * expf(src[s * W] - mm);
    const float gw = (gate && ex.gate_wide) ? sigmoidf_(ldf(gate + (long)b * ldg + h * V + ch)) : 1.f;
    stf(y + (long)b * ldy + h * V + ch, a * (gt * ex.out_scale) / ll * gw);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Mixture of experts.
//   moe_topk    : from the fp32 router logits z = W_r h (a product of the caller's): s = sigmoid(z), the `top` largest
//                 (ties: the lower index), weights s / (sum + 1e-20) * rscale (mode 2: the scores themselves, s * rscale);
//                 optionally counts the tokens of every expert.
//   pair kernels: few tokens (single-token steps): every (token, chosen expert) pair reads its expert's matrices —
//                 a = act(W_gate h) * (W_up h), then out[t] = sum_k weight_k W_down,k a_k in fp32.  `win` puts the weight on
//                 the expert's input instead: the pair reads weight_k * h (rounded to T) and the outputs are summed.
//   sort kernels: many tokens: rows are copied into a matrix sorted by expert (offsets from the counts), the experts
//                 run as dense products on their row ranges, and the fused residual kernel gathers the weighted sum.
// Expert matrices are stacked: wgu [E, 2*ff, n] (gate rows, then up rows), wd [E, n, ff].
// ------------------------------------------------------------------------------------------------------------------
// one warp per token over its fp32 router logits z [tokens, E] (+ bias [E] when given).  mode 0: scores sigmoid(z), weights
// score / (sum of the chosen scores + 1e-20) * rscale; mode 1: scores z, weights = softmax over the chosen logits, times rscale;
// mode 2: scores sigmoid(z), weights = the chosen scores as they are, times rscale
__global__ void moe_topk_kernel(const float* __restrict__ z, long ldz, const float* __restrict__ bias, int mode, int E, int top,
                                float rscale, int* __restrict__ idx, float* __restrict__ wts, int* __restrict__ counts, long tokens) {
  extern __shared__ float sm[];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const long tok = (long)blockIdx.x * nw + wib;
  float* sc = sm + (long)wib * E;
  if (tok >= tokens) return;                     // warps are independent below
  for (int e = lane; e < E; e += 32) {
    const float v = z[tok * ldz + e] + (bias ? bias[e] : 0.f);
    sc[e] = mode == 1 ? v : sigmoidf_(v);
  }
  __syncwarp();
  float sum = 0.f, mine_w = 0.f, first = 0.f; int mine_e = 0;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY; int be = 0x7fffffff;
    for (int e = lane; e < E; e += 32) { const float v = sc[e]; if (v > best) { best = v; be = e; } }
#pragma unroll
    for (int mk = 16; mk > 0; mk >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, mk);
      const int oe = __shfl_xor_sync(0xffffffffu, be, mk);
      if (ov > best || (ov == best && oe < be)) { best = ov; be = oe; }
    }
    if (k == 0) first = best;
    const float wk = mode != 1 ? best : expf(best - first);   // the first choice is the largest logit
    sum += wk;
    if (lane == k % 32) { mine_w = wk; mine_e = be; }
    if (lane == 0) sc[be] = -INFINITY;
    __syncwarp();
    if (k % 32 == 31 || k == top - 1) {          // flush up to 32 choices held one per lane
      const int k0 = k - (k % 32);
      if (lane <= k - k0) { idx[tok * top + k0 + lane] = mine_e; wts[tok * top + k0 + lane] = mine_w; }
    }
  }
  __syncwarp();
  const float inv = mode == 2 ? rscale : rscale / (mode == 0 ? sum + 1e-20f : sum);
  for (int k = lane; k < top; k += 32) {
    wts[tok * top + k] *= inv;
    if (counts) atomicAdd(counts + idx[tok * top + k], 1);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_pair_gateup_kernel(const T* __restrict__ h, long ldh, const T* __restrict__ wgu, const int* __restrict__ idx,
                       const float* __restrict__ wts, int win, T* __restrict__ a, int ff, int n, int top, int act, float limit) {
  extern __shared__ float sm[];
  const long pair = blockIdx.x;
  const long tok = pair / top;
  const int e = idx[pair];
  if (win) {
    const float wp = wts[pair];
    for (int i = threadIdx.x; i < n; i += blockDim.x) { T r; stf(&r, wp * ldf(h + tok * ldh + i)); sm[i] = ldf(&r); }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) sm[i] = ldf(h + tok * ldh + i);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int per = (ff + gridDim.y - 1) / gridDim.y;
  const int f0 = blockIdx.y * per, f1 = min(ff, f0 + per);
  const T* wg = wgu + (long)e * 2 * ff * n;
  for (int f = f0 + warp; f < f1; f += nw) {
    const float gv = warp_dot<T>(wg + (long)f * n, sm, n, lane);
    const float uv = warp_dot<T>(wg + (long)(ff + f) * n, sm, n, lane);
    if (lane == 0) stf(a + pair * ff + f, gated_apply(gv, uv, act, limit));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_pair_down_kernel(const T* __restrict__ a, const T* __restrict__ wd, const int* __restrict__ idx, const float* __restrict__ wts,
                     int win, float* __restrict__ out, int ff, int n, int top) {
  extern __shared__ float sm[];
  const long tok = blockIdx.x;
  for (int i = threadIdx.x; i < top * ff; i += blockDim.x) sm[i] = ldf(a + tok * top * ff + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int per = (n + gridDim.y - 1) / gridDim.y;
  const int c0 = blockIdx.y * per, c1 = min(n, c0 + per);
  for (int c = c0 + warp; c < c1; c += nw) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int e = idx[tok * top + k];
      acc += (win ? 1.f : wts[tok * top + k]) * warp_dot<T>(wd + ((long)e * n + c) * ff, sm + k * ff, ff, lane);
    }
    if (lane == 0) out[tok * n + c] = acc;
  }
}

// offsets[e] = first sorted row of expert e (offsets[E] = end of the last one); the per-expert cursors start at zero.
// With `align` > 1 every expert's range starts on a multiple of it, and tile_group[i] names the expert that owns rows
// [i*align, (i+1)*align) of the sorted matrix (-1: nobody; `tiles` entries) — the list a grouped GEMM schedules by.
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ cursor, int E, int align,
                                   int* __restrict__ tile_group, int tiles) {
  __shared__ int s_off[1025];
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at; s_off[e] = at; cursor[e] = 0;
      at += (counts[e] + align - 1) / align * align;
    }
    offsets[E] = at; s_off[E] = at;
  }
  __syncthreads();
  if (tile_group) {
    for (int i = threadIdx.x; i < tiles; i += blockDim.x) {
      const int row = i * align;
      int g = -1;
      for (int e = 0; e < E; ++e) if (row >= s_off[e] && row < s_off[e] + counts[e]) { g = e; break; }
      tile_group[i] = g;
    }
  }
}

template <typename T>
__global__ void moe_scatter_kernel(const T* __restrict__ h, long ldh, const int* __restrict__ idx, const int* __restrict__ offsets,
                                   int* __restrict__ cursor, int* __restrict__ pos, T* __restrict__ xs, int n, int top,
                                   const float* __restrict__ wts) {   // wts given: the copied row is wts[pair] * h
  __shared__ int where;
  const long pair = blockIdx.x;
  if (threadIdx.x == 0) {
    const int e = idx[pair];
    where = offsets[e] + atomicAdd(cursor + e, 1);
    pos[pair] = where;
  }
  __syncthreads();
  const T* src = h + (pair / top) * ldh;
  T* dst = xs + (long)where * n;
  constexpr int PER = 16 / sizeof(T);
  if (wts) {
    const float wp = wts[pair];
    if (sizeof(T) == 2 && n % 8 == 0 && ldh % 8 == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)xs & 15) == 0) {
      for (int i = threadIdx.x; i < n / 8; i += blockDim.x) {            // eight bf16 channels per 16-byte access
        uint4 raw = reinterpret_cast<const uint4*>(src)[i];
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p2[e]); p2[e] = __floats2bfloat162_rn(wp * f.x, wp * f.y); }
        reinterpret_cast<uint4*>(dst)[i] = raw;
      }
    } else {
      for (int i = threadIdx.x; i < n; i += blockDim.x) stf(dst + i, wp * ldf(src + i));
    }
  } else if (n % PER == 0 && ldh % PER == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)xs & 15) == 0) {
    for (int i = threadIdx.x; i < n / PER; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
  }
}

}  // namespace

// ====================================================================================================================
// launchers (C ABI; return 0, a CUDA error code, or -1 for sizes a kernel is not built for)
// ====================================================================================================================
#define LAUNCH_END() do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : (int)e_; } while (0)
typedef __nv_bfloat16 bf16;

extern "C" {

int lbk_embed_scale(const void* table, const int64_t* ids, float scale, float* x, long rows, int n, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  if (dtype) embed_scale_kernel<bf16><<<(unsigned)rows, 256, 0, s>>>((const bf16*)table, ids, scale, x, n);
  else embed_scale_kernel<float><<<(unsigned)rows, 256, 0, s>>>((const float*)table, ids, scale, x, n);
  LAUNCH_END();
}

int lbk_dyt_residual(float* x, const void* y, long ldy, int ydtype, const int* pos, const float* cw, int top, const void* pw,
                     const void* pb, const void* palpha, const void* nw, const void* nb, const void* nalpha, void* h, long ldh,
                     long rows, int n, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  int th = n >= 1024 ? 256 : 128;
  auto al = [](const void* p, int a) { return p == nullptr || ((uintptr_t)p & (a - 1)) == 0; };
  const bool vec = n % 4 == 0 && ldy % 4 == 0 && ldh % 4 == 0 && al(x, 16) && al(y, 16) && al(h, 16) && al(pw, 16) && al(pb, 16) &&
                   al(nw, 16) && al(nb, 16);
  if (vec) {
    th = n >= 2048 ? 256 : (n >= 512 ? 128 : 64);
#define DYTV(T, Ty) dyt_residual_vec4_kernel<T, Ty><<<(unsigned)rows, th, 0, s>>>(x, (const Ty*)y, ldy, pos, cw, top, (const T*)pw, \
    (const T*)pb, (const T*)palpha, (const T*)nw, (const T*)nb, (const T*)nalpha, (T*)h, ldh, n)
    if (dtype) { if (ydtype) DYTV(bf16, bf16); else DYTV(bf16, float); }
    else { if (ydtype) return -1; DYTV(float, float); }
#undef DYTV
    LAUNCH_END();
  }
#define DYT(T, Ty) dyt_residual_kernel<T, Ty><<<(unsigned)rows, th, 0, s>>>(x, (const Ty*)y, ldy, pos, cw, top, (const T*)pw, \
    (const T*)pb, (const T*)palpha, (const T*)nw, (const T*)nb, (const T*)nalpha, (T*)h, ldh, n)
  if (dtype) { if (ydtype) DYT(bf16, bf16); else DYT(bf16, float); }
  else { if (ydtype) return -1; DYT(float, float); }
#undef DYT
  LAUNCH_END();
}

int lbk_act_rows(const void* in, long ldi, void* out, long ldo, long rows, int n, int act, int gated, float limit, int dtype,
                 cudaStream_t s) {
  if (act == 5 && !gated) return -1;
  if (rows == 0 || n == 0) return 0;
  const long total = rows * n;
  if (dtype && n % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const long work = total / 8;
    const unsigned g8 = (unsigned)((work + 255) / 256 > 148 * 16 ? 148 * 16 : (work + 255) / 256);
    act_rows_vec8_kernel<<<g8, 256, 0, s>>>((const bf16*)in, ldi, (bf16*)out, ldo, rows, n, act, gated, limit);
    LAUNCH_END();
  }
  const unsigned grid = (unsigned)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  if (dtype) act_rows_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)in, ldi, (bf16*)out, ldo, rows, n, act, gated, limit);
  else act_rows_kernel<float><<<grid, 256, 0, s>>>((const float*)in, ldi, (float*)out, ldo, rows, n, act, gated, limit);
  LAUNCH_END();
}

int lbk_softcap(float* l, float cap, long total, cudaStream_t s) {
  if (total == 0) return 0;
  const unsigned grid = (unsigned)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  softcap_kernel<<<grid, 256, 0, s>>>(l, cap, total);
  LAUNCH_END();
}

int lbk_qk_prepare(void* q, long ldq, void* k, long ldk, const void* qw, const void* kw, const float* freq, float mscale, int rot,
                   int H, int G, int D, float eps, int full_norm, int unit_norm, const int* tok_seq, const int* seq_off,
                   const int* past, long tokens, int dtype, cudaStream_t s) {
  if (tokens == 0) return 0;
  if (D > QK_MAXD || rot > D || (rot & 1)) return -1;
  const size_t smem = (size_t)(rot + 32) * sizeof(float);
  if (dtype) qk_prepare_kernel<bf16><<<(unsigned)tokens, 128, smem, s>>>((bf16*)q, ldq, (bf16*)k, ldk, (const bf16*)qw, (const bf16*)kw,
      freq, mscale, rot, H, G, D, eps, full_norm, unit_norm, tok_seq, seq_off, past);
  else qk_prepare_kernel<float><<<(unsigned)tokens, 128, smem, s>>>((float*)q, ldq, (float*)k, ldk, (const float*)qw, (const float*)kw,
      freq, mscale, rot, H, G, D, eps, full_norm, unit_norm, tok_seq, seq_off, past);
  LAUNCH_END();
}

int lbk_kv_write(void* ring, void* first, const void* knew, const void* vnew, long ldn, const int* tok_seq, const int* seq_off,
                 const int* slots, const int* past, long tokens, int KC, int VC, int L, int nfirst, int dtype, cudaStream_t s) {
  if (tokens == 0) return 0;
  if (dtype) kv_write_kernel<bf16><<<(unsigned)tokens, 128, 0, s>>>((bf16*)ring, (bf16*)first, (const bf16*)knew, (const bf16*)vnew, ldn,
      tok_seq, seq_off, slots, past, KC, VC, L, nfirst);
  else kv_write_kernel<float><<<(unsigned)tokens, 128, 0, s>>>((float*)ring, (float*)first, (const float*)knew, (const float*)vnew, ldn,
      tok_seq, seq_off, slots, past, KC, VC, L, nfirst);
  LAUNCH_END();
}

int lbk_kv_gather(const void* ring, const void* first, const void* knew, const void* vnew, long ldn, const int* ext_seq,
                  const int* ext_off, const int* nsink, const int* cstart, const int* seq_off, const int* slots, const int* past,
                  void* ext, long rows, int KC, int VC, int L, int nfirst, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  if (dtype) kv_gather_kernel<bf16><<<(unsigned)rows, 128, 0, s>>>((const bf16*)ring, (const bf16*)first, (const bf16*)knew,
      (const bf16*)vnew, ldn, ext_seq, ext_off, nsink, cstart, seq_off, slots, past, (bf16*)ext, KC, VC, L, nfirst);
  else kv_gather_kernel<float><<<(unsigned)rows, 128, 0, s>>>((const float*)ring, (const float*)first, (const float*)knew,
      (const float*)vnew, ldn, ext_seq, ext_off, nsink, cstart, seq_off, slots, past, (float*)ext, KC, VC, L, nfirst);
  LAUNCH_END();
}

int lbk_masked_attention(const void* q, long ldq, const void* kbase, const void* vbase, long ldkv, const void* ring, const void* first,
                         int L, int nfirst, const int* ext_off, const int* nsink, const int* cstart, const int* slots,
                         const void* gate, long ldg, const int* tok_seq, const int* seq_off, const int* past, void* y, long ldy,
                         long tokens, int H, int G, int D, int V, int window, int chunk, int keep, float scale, float softcap,
                         int sink, int gate_wide, float out_scale, int dtype, cudaStream_t s) {
  if (tokens == 0) return 0;
  const AttnExtra ex{softcap, out_scale, sink, gate_wide};
  if (V > 32 * ATT_MAXV || G <= 0 || H % G) return -1;
  KvSource src{kbase, vbase, ldkv, ring, first, L, nfirst, G * (D + V), G * D, ext_off, nsink, cstart, slots};
  const int warps = 4;
  const long nwarps = tokens * H;
  const unsigned grid = (unsigned)((nwarps + warps - 1) / warps);
  const size_t smem = (size_t)warps * D * sizeof(float);
  if (dtype) masked_attention_kernel<bf16><<<grid, warps * 32, smem, s>>>((const bf16*)q, ldq, src, (const bf16*)gate, ldg, tok_seq,
      seq_off, past, (bf16*)y, ldy, tokens, H, G, D, V, window, chunk, keep, scale, ex);
  else masked_attention_kernel<float><<<grid, warps * 32, smem, s>>>((const float*)q, ldq, src, (const float*)gate, ldg, tok_seq,
      seq_off, past, (float*)y, ldy, tokens, H, G, D, V, window, chunk, keep, scale, ex);
  LAUNCH_END();
}

int lbk_moe_topk(const float* z, long ldz, const float* bias, int mode, int E, int top, float rscale, int* idx, float* wts, int* counts,
                 long tokens, cudaStream_t s) {
  if (tokens == 0) return 0;
  if (top > E || (size_t)E * sizeof(float) > 12 * 1024) return -1;
  const int warps = 4;
  moe_topk_kernel<<<(unsigned)((tokens + warps - 1) / warps), warps * 32, (size_t)warps * E * sizeof(float), s>>>(z, ldz, bias, mode, E, top, rscale,
                                                                                                               idx, wts, counts, tokens);
  LAUNCH_END();
}

int lbk_moe_pairs(const void* h, long ldh, const void* wgu, const void* wd, const int* idx, const float* wts, void* a, float* out,
                  long tokens, int ff, int n, int top, int act, float limit, int win, int dtype, cudaStream_t s) {
  if (tokens == 0) return 0;
  const size_t smem1 = (size_t)n * sizeof(float), smem2 = (size_t)top * ff * sizeof(float);
  if (smem1 > 200 * 1024 || smem2 > 200 * 1024) return -1;
  const long pairs = tokens * top;
  // enough blocks to fill the device with few pairs, never less than 8 rows per block
  int sy1 = (int)((148 * 4 + pairs - 1) / pairs); if (sy1 > (ff + 7) / 8) sy1 = (ff + 7) / 8; if (sy1 < 1) sy1 = 1;
  int sy2 = (int)((148 * 4 + tokens - 1) / tokens); if (sy2 > (n + 7) / 8) sy2 = (n + 7) / 8; if (sy2 < 1) sy2 = 1;
  if (dtype) {
    if (smem1 > 48 * 1024) cudaFuncSetAttribute(moe_pair_gateup_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (smem2 > 48 * 1024) cudaFuncSetAttribute(moe_pair_down_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    moe_pair_gateup_kernel<bf16><<<dim3((unsigned)pairs, sy1), 256, smem1, s>>>((const bf16*)h, ldh, (const bf16*)wgu, idx, wts, win, (bf16*)a, ff, n, top, act, limit);
    moe_pair_down_kernel<bf16><<<dim3((unsigned)tokens, sy2), 256, smem2, s>>>((const bf16*)a, (const bf16*)wd, idx, wts, win, out, ff, n, top);
  } else {
    if (smem1 > 48 * 1024) cudaFuncSetAttribute(moe_pair_gateup_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (smem2 > 48 * 1024) cudaFuncSetAttribute(moe_pair_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    moe_pair_gateup_kernel<float><<<dim3((unsigned)pairs, sy1), 256, smem1, s>>>((const float*)h, ldh, (const float*)wgu, idx, wts, win, (float*)a, ff, n, top, act, limit);
    moe_pair_down_kernel<float><<<dim3((unsigned)tokens, sy2), 256, smem2, s>>>((const float*)a, (const float*)wd, idx, wts, win, out, ff, n, top);
  }
  LAUNCH_END();
}

int lbk_moe_sort(const void* h, long ldh, const int* idx, const int* counts, int* offsets, int* cursor, int* pos, void* xs, long tokens,
                 int E, int n, int top, int align, int* tile_group, int tiles, const float* wts, int dtype, cudaStream_t s) {
  if (tokens == 0) return 0;
  if (E > 1024 || align < 1) return -1;
  moe_offsets_kernel<<<1, 256, 0, s>>>(counts, offsets, cursor, E, align, tile_group, tiles);
  const unsigned pairs = (unsigned)(tokens * top);
  if (dtype) moe_scatter_kernel<bf16><<<pairs, 128, 0, s>>>((const bf16*)h, ldh, idx, offsets, cursor, pos, (bf16*)xs, n, top, wts);
  else moe_scatter_kernel<float><<<pairs, 128, 0, s>>>((const float*)h, ldh, idx, offsets, cursor, pos, (float*)xs, n, top, wts);
  LAUNCH_END();
}

int lbk_masked_attention_mma(const void* q, long ldq, const void* kbase, const void* vbase, long ldkv, const int* ext_off,
                             const int* nsink, const int* cstart, const void* gate, long ldg, const int* qt_seq, const int* qt_start,
                             int n_qtiles, const int* seq_off, const int* past, void* y, long ldy, int H, int G, int D, int V,
                             int window, int chunk, int keep, float scale, float softcap, int sink, int gate_wide, float out_scale,
                             cudaStream_t s) {
  if (n_qtiles == 0) return 0;
  if (D != V || G <= 0 || H % G) return -1;
  const AttnExtra ex{softcap, out_scale, sink, gate_wide};
  const dim3 grid((unsigned)n_qtiles, (unsigned)H);
#define MMA_CASE(DD) case DD: { \
    constexpr int smem = 2 * 64 * (2 * DD + 16) * 2; \
    static bool once = false; \
    if (!once) { cudaFuncSetAttribute(masked_attention_mma_kernel<DD, DD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); once = true; } \
    masked_attention_mma_kernel<DD, DD><<<grid, 128, smem, s>>>((const bf16*)q, ldq, (const bf16*)kbase, \
    (const bf16*)vbase, ldkv, ext_off, nsink, cstart, (const bf16*)gate, ldg, qt_seq, qt_start, seq_off, past, (bf16*)y, ldy, H, G, \
    window, chunk, keep, scale, ex); } break
  switch (D) {
    MMA_CASE(32); MMA_CASE(48); MMA_CASE(64); MMA_CASE(96); MMA_CASE(128);
    default: return -1;
  }
#undef MMA_CASE
  LAUNCH_END();
}

int lbk_ring_decode(const void* q, long ldq, const void* ring, const void* first, int L, int nfirst, const int* slots, const int* past,
                    const void* gate, long ldg, void* y, long ldy, float* part, int B, int H, int G, int D, int V, int window,
                    int chunk, int keep, float scale, int splits, float softcap, int sink, int gate_wide, float out_scale, int dtype,
                    cudaStream_t s) {
  if (B == 0) return 0;
  const AttnExtra ex{softcap, out_scale, sink, gate_wide};
  if (G <= 0 || H % G || H / G > DEC_MAXR || V > 32 * DEC_MAXVL || splits < 1) return -1;
  const int R = H / G;
  const size_t smem = ((size_t)R * D + 4 * (size_t)R * (V + 2)) * sizeof(float);
  if (smem > 48 * 1024) return -1;
  const dim3 grid((unsigned)B, (unsigned)G, (unsigned)splits);
  const int C = G * (D + V);
  if (dtype) {
    const int vec = (D % 8 == 0 && C % 8 == 0 && ((uintptr_t)ring & 15) == 0 && ((uintptr_t)first & 15) == 0) ? 1 : 0;
    ring_decode_kernel<bf16><<<grid, 128, smem, s>>>((const bf16*)q, ldq, (const bf16*)ring, (const bf16*)first, L, nfirst, slots, past,
                                                     part, H, G, D, V, window, chunk, keep, scale, splits, vec, softcap);
    ring_decode_merge_kernel<bf16><<<dim3((unsigned)B, (unsigned)H), 64, 0, s>>>(part, (const bf16*)gate, ldg, (bf16*)y, ldy, H, V, splits, ex);
  } else {
    const int vec = (D % 8 == 0 && C % 4 == 0 && ((uintptr_t)ring & 15) == 0 && ((uintptr_t)first & 15) == 0) ? 1 : 0;
    ring_decode_kernel<float><<<grid, 128, smem, s>>>((const float*)q, ldq, (const float*)ring, (const float*)first, L, nfirst, slots,
                                                      past, part, H, G, D, V, window, chunk, keep, scale, splits, vec, softcap);
    ring_decode_merge_kernel<float><<<dim3((unsigned)B, (unsigned)H), 64, 0, s>>>(part, (const float*)gate, ldg, (float*)y, ldy, H, V, splits, ex);
  }
  LAUNCH_END();
}

}  // extern "C"
