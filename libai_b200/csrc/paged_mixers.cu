// Kernels of decoders whose attention layers see the whole past of a sequence through a paged key/value cache:
//   * post-norm residual: x <- rmsnorm(alpha * x + sublayer output) * (1 + w) on the fp32 residual, with the compute-dtype copy
//     that the next sublayer's products read (the sublayer output may be a dense matrix plus rows gathered from a matrix of
//     expert outputs sorted by expert);
//   * query / key / value preparation in one pass: per-channel causal convolution over time (tails carried per sequence),
//     per-head RMS norm of queries and keys with a weight shared by the heads, rotary positions on the leading channels,
//     unit-RMS values, keys and values written into their page;
//   * softmax attention over the pages with two optional extras: the heads' scores are mixed by a matrix before the softmax
//     ("talking heads": s'_h = sum_g talk[h, g] s_g) and the softmax denominator carries exp(sink_h) of a learned number per
//     head that has no key and no value.  One kernel serves prompts (tiles of queries, all heads of a tile in one block because
//     the mix couples them) and single-token steps (the keys of a sequence cut into parts, merged by a second kernel).
//
// Conventions (the ragged-batch descriptor of the other mixer libraries).  A step carries B sequences; sequence b brings
// n_b = seq_off[b+1]-seq_off[b] new tokens packed at rows seq_off[b].., has past[b] tokens already in its state, which lives in
// slot slots[b].  A cache row is [G*D keys | G*V values] (C numbers) of one position; position p of a sequence lives in row
// p % page_size of page table[slot * max_pages + p / page_size] of the pool [pages, page_size, C].  Activations are `T` (float
// or bf16); scores, softmax, norms, angles and the residual are fp32 in both.  Built WITHOUT fast-math.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace {
typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

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

// ------------------------------------------------------------------------------------------------------------------
// Post-norm residual.  v = alpha * x + y1 + y2', r = 1 / sqrt(mean(v^2) + eps), out = v * r * (1 + w); `xout` (fp32, may
// be x itself) and `h` (T) receive it when given.  y1 [rows, n] (Ty) and y2 (fp32) are optional; with `pos` [rows, top]
// y2' = sum_k cw[r, k] * y2[pos[r, k]] (cw absent: 1), else y2' = y2[r].  One block per row; the row is staged in shared memory.
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float4 ld4f(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4f(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
  return make_float4(__low2float(h2[0]), __high2float(h2[0]), __low2float(h2[1]), __high2float(h2[1]));
}
__device__ __forceinline__ void st4f(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4f(bf16* p, float4 v) {
  uint2 o;
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&o);
  h2[0] = __floats2bfloat162_rn(v.x, v.y); h2[1] = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = o;
}

// four channels per thread and access (every row and pointer aligned to four elements); the row stays in registers when it
// fits (at most ITEMS quadruples per thread), so nothing is staged
template <typename T, typename Ty, int ITEMS>
__global__ void postnorm_residual_vec_kernel(const float* xin, float* xout, const Ty* __restrict__ y1, long ldy1, const float* __restrict__ y2,
                                             long ldy2, const int* __restrict__ pos, const float* __restrict__ cw, int top, float alpha,
                                             const T* __restrict__ w, float eps, T* __restrict__ h, long ldh, int n) {
  __shared__ float red[32];
  const long row = blockIdx.x;
  const int quads = n / 4;
  float4 v[ITEMS];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const int i = (threadIdx.x + it * blockDim.x) * 4;
    v[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < quads * 4) {
      float4 a = ld4f(xin + row * n + i);
      a.x *= alpha; a.y *= alpha; a.z *= alpha; a.w *= alpha;
      if (y1) { const float4 b = ld4f(y1 + row * ldy1 + i); a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
      if (y2) {
        if (pos) {
          for (int k = 0; k < top; ++k) {
            const float c = cw ? cw[row * top + k] : 1.f;
            const float4 b = ld4f(y2 + (long)pos[row * top + k] * ldy2 + i);
            a.x += c * b.x; a.y += c * b.y; a.z += c * b.z; a.w += c * b.w;
          }
        } else {
          const float4 b = ld4f(y2 + row * ldy2 + i);
          a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
      }
      v[it] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)n + eps);
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const int i = (threadIdx.x + it * blockDim.x) * 4;
    if (i < quads * 4) {
      const float4 ww = ld4f(w + i);
      const float4 o = make_float4(v[it].x * r * (1.f + ww.x), v[it].y * r * (1.f + ww.y), v[it].z * r * (1.f + ww.z), v[it].w * r * (1.f + ww.w));
      if (xout) st4f(xout + row * n + i, o);
      if (h) st4f(h + row * ldh + i, o);
    }
  }
}

template <typename T, typename Ty>
__global__ void postnorm_residual_kernel(const float* xin, float* xout, const Ty* __restrict__ y1, long ldy1, const float* __restrict__ y2,
                                         long ldy2, const int* __restrict__ pos, const float* __restrict__ cw, int top, float alpha,
                                         const T* __restrict__ w, float eps, T* __restrict__ h, long ldh, int n) {
  extern __shared__ float sm[];
  __shared__ float red[32];
  const long row = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = alpha * xin[row * n + i];
    if (y1) v += ldf(y1 + row * ldy1 + i);
    if (y2) {
      if (pos) {
        for (int k = 0; k < top; ++k) v += (cw ? cw[row * top + k] : 1.f) * y2[(long)pos[row * top + k] * ldy2 + i];
      } else {
        v += y2[row * ldy2 + i];
      }
    }
    sm[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float o = sm[i] * r * (1.f + ldf(w + i));
    if (xout) xout[row * n + i] = o;
    if (h) stf(h + row * ldh + i, o);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Query / key / value preparation.  One warp per (token, head unit): the H query heads, then the G key heads, then the
// G value heads.  u = the projections (three column slices with one row stride); y_t = sum_j w[c, j] u_(t - taps + 1 + j)
// with zeros before the sequence's start, earlier steps' rows taken from `tail` [slots, taps-1, C] (row r = position
// past - (taps-1) + r; channels [q | k | v]).  Queries and keys: y / sqrt(mean(y^2) + eps) * norm[c] over the head, then the
// pair (c, c + half), c < half, is turned by the angle position * freq[c].  Values: y / sqrt(mean(y^2) + eps).  Queries go to
// qout, keys and values into the sequence's page row.  The tails are rewritten by a second kernel (the first tokens of a step
// read what the last ones would overwrite).
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int VEC> struct VecLd;
template <typename T> struct VecLd<T, 1> { static __device__ __forceinline__ void ld(const T* p, float (&f)[1]) { f[0] = ldf(p); } };
template <> struct VecLd<float, 4> {
  static __device__ __forceinline__ void ld(const float* p, float (&f)[4]) { const float4 a = *reinterpret_cast<const float4*>(p); f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; }
};
template <> struct VecLd<bf16, 4> {
  static __device__ __forceinline__ void ld(const bf16* p, float (&f)[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    f[0] = __low2float(h2[0]); f[1] = __high2float(h2[0]); f[2] = __low2float(h2[1]); f[3] = __high2float(h2[1]);
  }
};

__device__ __forceinline__ void st4v(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
__device__ __forceinline__ void st4v(bf16* p, float a, float b, float c, float d) {
  uint2 o;
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&o);
  h2[0] = __floats2bfloat162_rn(a, b); h2[1] = __floats2bfloat162_rn(c, d);
  *reinterpret_cast<uint2*>(p) = o;
}

// VEC consecutive channels per lane (4: every row slice and pointer is aligned to 4 elements; 1: anything)
template <typename T, int VEC>
__global__ void __launch_bounds__(128)
conv_qkv_prepare_kernel(const T* __restrict__ qin, const T* __restrict__ kin, const T* __restrict__ vin, long ld,
                        const T* __restrict__ wq, const T* __restrict__ wk, const T* __restrict__ wv, int taps,
                        const T* __restrict__ tail, const T* __restrict__ qn, const T* __restrict__ kn, const float* __restrict__ freq,
                        int half, float eps, T* __restrict__ qout, long ldqo, T* __restrict__ pool, const int* __restrict__ table,
                        int max_pages, int page_size, const int* __restrict__ tok_seq, const int* __restrict__ seq_off,
                        const int* __restrict__ slots, const int* __restrict__ past, long tokens, int H, int G, int D, int V, int W) {
  extern __shared__ float sm[];
  const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long unit = (long)blockIdx.x * (blockDim.x >> 5) + wib;
  const int units = H + 2 * G;
  if (unit >= tokens * units) return;            // warps are independent
  float* buf = sm + (long)wib * W;
  const long tok = unit / units;
  const int u = (int)(unit - tok * units);
  const int b = tok_seq[tok], s0 = seq_off[b], t = (int)(tok - s0), pb = past[b], p = pb + t, slot = slots[b];
  const int kind = u < H ? 0 : (u < H + G ? 1 : 2);
  const int hh = kind == 0 ? u : (kind == 1 ? u - H : u - H - G);
  const int n = kind == 2 ? V : D;
  const int C = H * D + G * D + G * V, R = taps - 1;
  const T* in = kind == 0 ? qin + hh * D : (kind == 1 ? kin + hh * D : vin + hh * V);
  const T* cw = (kind == 0 ? wq : (kind == 1 ? wk : wv)) + (long)hh * n * taps;
  const int coff = kind == 0 ? hh * D : (kind == 1 ? H * D + hh * D : H * D + G * D + hh * V);
  float ss = 0.f;
  const bool w4 = VEC == 4 && taps == 4 && (reinterpret_cast<uintptr_t>(cw) % (4 * sizeof(T))) == 0;
  for (int c = lane * VEC; c < n; c += 32 * VEC) {
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    if (w4) {                                    // the four taps of a channel are one aligned load
      float wt[VEC][4];
#pragma unroll
      for (int e = 0; e < VEC; ++e) VecLd<T, VEC == 4 ? 4 : 1>::ld(cw + (long)(c + e) * 4, reinterpret_cast<float (&)[VEC == 4 ? 4 : 1]>(wt[e]));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int lt = t - 3 + j;
        float uv[VEC];
        if (lt >= 0) VecLd<T, VEC>::ld(in + (long)(s0 + lt) * ld + c, uv);
        else if (pb + lt >= 0) VecLd<T, VEC>::ld(tail + ((long)slot * 3 + (3 + lt)) * C + coff + c, uv);
        else continue;
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] += wt[e][j] * uv[e];
      }
    } else
    for (int j = 0; j < taps; ++j) {
      const int lt = t - R + j;
      float uv[VEC];
      if (lt >= 0) VecLd<T, VEC>::ld(in + (long)(s0 + lt) * ld + c, uv);
      else if (pb + lt >= 0) VecLd<T, VEC>::ld(tail + ((long)slot * R + (R + lt)) * C + coff + c, uv);
      else continue;
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] += ldf(cw + (long)(c + e) * taps + j) * uv[e];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) { buf[c + e] = acc[e]; ss += acc[e] * acc[e]; }
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)n + eps);
  __syncwarp();
  T* krow = pool + ((long)table[(long)slot * max_pages + p / page_size] * page_size + p % page_size) * (long)(G * D + G * V);
  if (kind == 2) {
    T* dv = krow + G * D + hh * V;
    if (VEC == 4 && (reinterpret_cast<uintptr_t>(dv) % (4 * sizeof(T))) == 0) {
      for (int c = lane * 4; c < n; c += 128) st4v(dv + c, buf[c] * r, buf[c + 1] * r, buf[c + 2] * r, buf[c + 3] * r);
    } else {
      for (int c = lane; c < n; c += 32) stf(dv + c, buf[c] * r);
    }
    return;
  }
  const T* nw = kind == 0 ? qn : kn;
  T* dst = kind == 0 ? qout + tok * ldqo + hh * D : krow + hh * D;
  int plain = 2 * half;                           // first channel that is stored by the scalar loop's pass-through branch
  if (VEC == 4 && half % 2 == 0 && (reinterpret_cast<uintptr_t>(dst) % (4 * sizeof(T))) == 0) {
    for (int c = 2 * half + lane * 4; c < n; c += 128)
      st4v(dst + c, buf[c] * r * ldf(nw + c), buf[c + 1] * r * ldf(nw + c + 1), buf[c + 2] * r * ldf(nw + c + 2), buf[c + 3] * r * ldf(nw + c + 3));
    plain = n;
  }
  for (int c = lane; c < (plain < n ? n : 2 * half); c += 32) {   // a lane below `half` turns its pair (c, c + half) once and writes both
    if (c < half) {
      const float a = buf[c] * r * ldf(nw + c), bq = buf[c + half] * r * ldf(nw + c + half);
      float sn, cs;
      sincosf((float)p * freq[c], &sn, &cs);
      stf(dst + c, a * cs - bq * sn);
      stf(dst + c + half, bq * cs + a * sn);
    } else if (c >= 2 * half) {
      stf(dst + c, buf[c] * r * ldf(nw + c));
    }
  }
}

// tail[slot][r] <- the projection at position past + n - (taps-1) + r: a row of this step, or an older tail row
template <typename T>
__global__ void conv_tail_update_kernel(const T* __restrict__ qin, const T* __restrict__ kin, const T* __restrict__ vin, long ld,
                                        T* __restrict__ tail, int R, const int* __restrict__ seq_off, const int* __restrict__ slots,
                                        const int* __restrict__ past, int HD, int GD, int GV) {
  const int b = blockIdx.y;
  const int C = HD + GD + GV;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s0 = seq_off[b], n = seq_off[b + 1] - s0, pb = past[b];
  T* tl = tail + (long)slots[b] * R * C + c;
  const T* in = c < HD ? qin + c : (c < HD + GD ? kin + (c - HD) : vin + (c - HD - GD));
  for (int r = 0; r < R; ++r) {                  // ascending: an older row moves down before its place is rewritten
    const int lt = n - R + r;
    T val;
    if (lt >= 0) val = in[(long)(s0 + lt) * ld];
    else if (pb + lt >= 0) val = tl[(long)(r + n) * C];
    else stf(&val, 0.f);
    tl[(long)r * C] = val;
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Attention over the pages.  Block (tile, part): QT consecutive new tokens of one sequence (qt_seq / qt_start name the tile),
// all heads, the keys [part * len, (part + 1) * len) of the positions 0 .. the tile's last query, KT at a time:
//   A  raw scores of every (head, key, query) from Q and the key tile in shared memory (a thread: one head and key, QT queries);
//   B  the mix over heads and the causal mask;
//   C  online softmax per (head, query) row: a warp per row;
//   D  O <- O * correction + P V (a thread: one (head, channel), QT queries).
// nparts == 1: the result (with the sink in the denominator, times out_scale) goes to y; otherwise the running maximum, sum
// and unnormalised O of the part go to `part` [rows, nparts, H, V + 2] and the merge kernel finishes.
// ------------------------------------------------------------------------------------------------------------------
template <typename T, int QT>
__global__ void __launch_bounds__(256)
talk_attention_kernel(const T* __restrict__ q, long ldq, const T* __restrict__ pool, const int* __restrict__ table, int max_pages,
                      int page_size, const float* __restrict__ talk, const float* __restrict__ sink, const int* __restrict__ qt_seq,
                      const int* __restrict__ qt_start, const int* __restrict__ seq_off, const int* __restrict__ slots,
                      const int* __restrict__ past, T* __restrict__ y, long ldy, float* __restrict__ part, int nparts, int KT, int H,
                      int G, int D, int V, float scale, float out_scale) {
  extern __shared__ float sm[];
  const int HD = H * D, HV = H * V, GD = G * D, GV = G * V, KP = GD + 1, rep = H / G;
  float* Qs = sm;                       // [QT][HD]
  float* Os = Qs + QT * HD;             // [QT][HV]
  float* Ks = Os + QT * HV;             // [KT][GD + 1]
  float* Vs = Ks + KT * KP;             // [KT][GV]
  float* S0 = Vs + KT * GV;             // [H][QT][KT] raw scores
  float* S1 = S0 + H * QT * KT;         // [H][QT][KT] mixed scores, then probabilities
  float* Ms = S1 + H * QT * KT;         // [H][QT] running maximum
  float* Ls = Ms + H * QT;              // [H][QT] running sum
  float* Cs = Ls + H * QT;              // [H][QT] correction of this tile
  float* Ts = Cs + H * QT;              // [H][H]
  const int tid = threadIdx.x, nth = blockDim.x, warp = tid >> 5, lane = tid & 31, nw = nth >> 5;
  const int b = qt_seq[blockIdx.x], t0 = qt_start ? qt_start[blockIdx.x] : 0;
  const int s0 = seq_off[b], nq = min(QT, seq_off[b + 1] - s0 - t0), pos0 = past[b] + t0;
  const long row0 = s0 + t0;
  const long slot = slots[b];
  const int kall = pos0 + nq;                                   // keys the tile's last query sees
  int len = (kall + nparts - 1) / nparts;
  len = (len + KT - 1) / KT * KT;
  const int kbeg = blockIdx.y * len, kend = min(kall, kbeg + len);
  const long C = GD + GV;
  const bool vec8 = GD % 8 == 0 && GV % 8 == 0 && (reinterpret_cast<uintptr_t>(pool) & 15) == 0;

  for (int i = tid; i < QT * HD; i += nth) {
    const int qi = i / HD, c = i - qi * HD;
    Qs[i] = qi < nq ? ldf(q + (row0 + qi) * ldq + c) : 0.f;
  }
  for (int i = tid; i < QT * HV; i += nth) Os[i] = 0.f;
  for (int i = tid; i < H * QT; i += nth) { Ms[i] = -INFINITY; Ls[i] = 0.f; }
  if (talk) for (int i = tid; i < H * H; i += nth) Ts[i] = talk[i];

  for (int k0 = kbeg; k0 < kend; k0 += KT) {
    __syncthreads();                                            // the previous tile's phase D has read Ks / Vs / S1
    for (int j = warp; j < KT; j += nw) {
      const int kp = k0 + j;
      if (kp < kend) {
        const T* rowp = pool + ((long)table[slot * max_pages + kp / page_size] * page_size + kp % page_size) * C;
        if (sizeof(T) == 2 && vec8) {             // eight bf16 channels per lane and load
          for (int c = lane * 8; c < GD; c += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(rowp + c);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) { Ks[j * KP + c + 2 * e] = __low2float(h2[e]); Ks[j * KP + c + 2 * e + 1] = __high2float(h2[e]); }
          }
          for (int c = lane * 8; c < GV; c += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(rowp + GD + c);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) { Vs[j * GV + c + 2 * e] = __low2float(h2[e]); Vs[j * GV + c + 2 * e + 1] = __high2float(h2[e]); }
          }
        } else {
          for (int c = lane; c < GD; c += 32) Ks[j * KP + c] = ldf(rowp + c);
          for (int c = lane; c < GV; c += 32) Vs[j * GV + c] = ldf(rowp + GD + c);
        }
      } else {
        for (int c = lane; c < GD; c += 32) Ks[j * KP + c] = 0.f;
        for (int c = lane; c < GV; c += 32) Vs[j * GV + c] = 0.f;
      }
    }
    __syncthreads();
    // A: raw scores
    for (int item = tid; item < H * KT; item += nth) {
      const int g = item / KT, j = item - g * KT;
      const float* kr = Ks + j * KP + (g / rep) * D;
      const float* qr = Qs + g * D;
      float acc[QT];
#pragma unroll
      for (int i = 0; i < QT; ++i) acc[i] = 0.f;
      for (int d = 0; d < D; ++d) {
        const float kv = kr[d];
#pragma unroll
        for (int i = 0; i < QT; ++i) acc[i] += qr[i * HD + d] * kv;
      }
#pragma unroll
      for (int i = 0; i < QT; ++i) S0[(g * QT + i) * KT + j] = acc[i] * scale;
    }
    __syncthreads();
    // B: mix over heads, causal mask
    for (int item = tid; item < H * QT * KT; item += nth) {
      const int j = item % KT, hi = item / KT, i = hi % QT, h = hi / QT;
      float v;
      if (talk) {
        v = 0.f;
        for (int g = 0; g < H; ++g) v += Ts[h * H + g] * S0[(g * QT + i) * KT + j];
      } else {
        v = S0[item];
      }
      const int kp = k0 + j;
      S1[item] = (i < nq && kp < kend && kp <= pos0 + i) ? v : -INFINITY;
    }
    __syncthreads();
    // C: online softmax, a warp per (head, query) row
    for (int rrow = warp; rrow < H * QT; rrow += nw) {
      float* sr = S1 + rrow * KT;
      float mx = -INFINITY;
      for (int j = lane; j < KT; j += 32) mx = fmaxf(mx, sr[j]);
      mx = warp_max(mx);
      const float mo = Ms[rrow], mn = fmaxf(mo, mx);
      float sum = 0.f;
      for (int j = lane; j < KT; j += 32) {
        const float pj = mn == -INFINITY ? 0.f : expf(sr[j] - mn);
        sr[j] = pj;
        sum += pj;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float corr = mo == -INFINITY ? 0.f : expf(mo - mn);     // nothing accumulated yet: O and the sum are zero
        Cs[rrow] = corr;
        Ls[rrow] = Ls[rrow] * corr + sum;
        Ms[rrow] = mn;
      }
    }
    __syncthreads();
    // D: O <- O * corr + P V
    for (int item = tid; item < HV; item += nth) {
      const int h = item / V, v = item - h * V;
      const float* vr = Vs + (h / rep) * V + v;
      const float* pr = S1 + h * QT * KT;
      float acc[QT];
#pragma unroll
      for (int i = 0; i < QT; ++i) acc[i] = Os[i * HV + item] * Cs[h * QT + i];
      for (int j = 0; j < KT; ++j) {
        const float vv = vr[j * GV];
#pragma unroll
        for (int i = 0; i < QT; ++i) acc[i] += pr[i * KT + j] * vv;
      }
#pragma unroll
      for (int i = 0; i < QT; ++i) Os[i * HV + item] = acc[i];
    }
  }
  __syncthreads();
  if (nparts == 1) {
    for (int item = tid; item < nq * HV; item += nth) {
      const int i = item / HV, hv = item - i * HV, h = hv / V;
      const float m = Ms[h * QT + i];
      float l = Ls[h * QT + i], o = Os[i * HV + hv];
      if (sink) {
        const float mm = fmaxf(m, sink[h]), e = expf(m - mm);
        l = l * e + expf(sink[h] - mm);
        o *= e;
      }
      stf(y + (row0 + i) * ldy + hv, o / l * out_scale);
    }
  } else {
    for (int item = tid; item < nq * H * (V + 2); item += nth) {
      const int i = item / (H * (V + 2)), rest = item - i * H * (V + 2), h = rest / (V + 2), c = rest - h * (V + 2);
      float* dst = part + (((row0 + i) * nparts + blockIdx.y) * H + h) * (long)(V + 2);
      dst[c] = c == 0 ? Ms[h * QT + i] : (c == 1 ? Ls[h * QT + i] : Os[i * HV + h * V + c - 2]);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Tensor-core form of the prompt tiling for bf16 with equal key and value head sizes DH (mma.m16n8k16, ldmatrix,
// cp.async).  A block takes 16 consecutive queries of one sequence and all heads, one warp per head, 32 keys at a time:
//   1  warp h: raw scores Q_h K^T of its head on the tensor cores, times scale, as fp32 into shared memory;
//   2  the mix over heads on the fp32 pipe: warp w takes HB output heads and 16 / HB of the rows, i.e. 16 (head, row) pairs; a
//      lane owns one pair and one half of the 32 keys, keeps its head's row of `talk` in registers and its 16 mixed scores in
//      registers, so that the row maximum and sum are in-lane loops plus one exchange between the two halves; causal mask;
//      online softmax (running maximum and sum in the lane); probabilities as bf16 and the correction factors into shared
//      memory.  With heads in groups of four (HB = 4) a lane instead owns one row, four keys and the
//      four heads of its warp, with `talk` read from shared memory, so that a loaded raw score feeds four multiply-adds (the
//      shared-memory loads of the mix, H per mixed score otherwise, are what bounds this phase at 16 heads);
//   3  warp h: O_h <- O_h * correction + P_h V on the tensor cores, O in registers.
// The key tile of the next step is fetched (cp.async) while 2 and 3 run, the value tile of this step while 1 and 2 run.
// HP is the head count padded to 8 or 16 (the size of the register arrays); QREG keeps a head's query fragments in registers.
// ------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(a), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N)); }

constexpr int TM_Q = 16, TM_K = 32, TM_SRS = TM_K + 1;           // queries, keys per tile; row stride of the fp32 scores (odd: rows fall into different banks)
constexpr int TM_PRS = TM_K + 8, TM_PHS = TM_Q * TM_PRS + 8;     // row and head stride of the bf16 probabilities

template <int DH, int HP, int HB, bool QREG>
__global__ void __launch_bounds__(HP * 32, 1)
talk_attention_mma_kernel(const bf16* __restrict__ q, long ldq, const bf16* __restrict__ pool, const int* __restrict__ table,
                          int max_pages, int page_size, const float* __restrict__ talk, const float* __restrict__ sink,
                          const int* __restrict__ qt_seq, const int* __restrict__ qt_start, const int* __restrict__ seq_off,
                          const int* __restrict__ slots, const int* __restrict__ past, bf16* __restrict__ y, long ldy, int H, int G,
                          float scale, float out_scale) {
  extern __shared__ __align__(16) unsigned char smraw[];
  constexpr int KS = DH / 16, NT = DH / 8, RPW = TM_Q / HB;
  const int GD = G * DH, C = 2 * GD, rep = H / G;
  const int KRS = GD + 8;                       // bf16 elements per row of the key / value tiles
  const int QRS = H * DH + 8;
  constexpr int PRS = TM_PRS, PHS = TM_PHS;
  bf16* Ks = reinterpret_cast<bf16*>(smraw);
  bf16* Vs = Ks + TM_K * KRS;
  bf16* Qs = Vs + TM_K * KRS;
  bf16* Ps = Qs + TM_Q * QRS;                   // [H][16][PRS]
  float* S0 = reinterpret_cast<float*>(Ps + H * PHS);          // [H][16][TM_SRS]
  float* Cs = S0 + H * TM_Q * TM_SRS;           // [H][16] correction of this tile, then the final maximum
  float* Ls = Cs + H * TM_Q;                    // [H][16] final sum
  float* Tt = Ls + H * TM_Q;                    // [H][H] `talk` transposed: Tt[g][h]
  constexpr bool WIDE = HB == 4;                // phase 2 with four heads per lane
  const int tid = threadIdx.x, nth = blockDim.x, warp = tid >> 5, lane = tid & 31;
  const int b = qt_seq[blockIdx.x], t0 = qt_start ? qt_start[blockIdx.x] : 0;
  const int s0 = seq_off[b], nq = min(TM_Q, seq_off[b + 1] - s0 - t0), pos0 = past[b] + t0;
  const long row0 = s0 + t0;
  const long slot = slots[b];
  const int kend = pos0 + nq;
  const int h = warp, kvh = h / rep;

  // 32 cache rows, columns [coff, coff + GD), 16 bytes per copy: a thread keeps its column chunk and walks the rows (the
  // launcher makes the block a multiple of the chunks per row); a page size that is a power of two is a shift
  const int per = GD / 8, jstep = nth / per, j0 = tid / per, cc = (tid - j0 * per) * 8;
  const int pshift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
  auto load_rows = [&](bf16* dst, int k0, int coff) {
    for (int j = j0; j < TM_K; j += jstep) {
      const int kp = k0 + j;
      if (kp < kend) {
        const int pg = pshift >= 0 ? kp >> pshift : kp / page_size;
        const bf16* rowp = pool + ((long)table[slot * max_pages + pg] * page_size + (kp - pg * page_size)) * (long)C + coff;
        cp_async16(dst + j * KRS + cc, rowp + cc);
      } else {
        *reinterpret_cast<uint4*>(dst + j * KRS + cc) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  load_rows(Ks, 0, 0);
  cp_async_commit();
  {
    const int per = H * DH / 8;
    for (int i = tid; i < TM_Q * per; i += nth) {
      const int r = i / per, c = (i - r * per) * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < nq) v = *reinterpret_cast<const uint4*>(q + (row0 + r) * ldq + c);
      *reinterpret_cast<uint4*>(Qs + r * QRS + c) = v;
    }
  }
  // phase-2 role of this lane: pair p = lane % 16 of the warp's 16 (head, row) pairs — head grp * HB + p / RPW, row
  // rs * RPW + p % RPW — and the keys [16 * (lane / 16), + 16) of the tile
  const int grp = warp / HB, rs = warp % HB;
  const int h2 = grp * HB + (lane & 15) / RPW, i2 = rs * RPW + (lane & 15) % RPW, half = lane >> 4;
  float Tr[HP];
#pragma unroll
  for (int g = 0; g < HP; ++g) Tr[g] = (g < H && h2 < H) ? (talk ? talk[h2 * H + g] : (g == h2 ? 1.f : 0.f)) : 0.f;
  float m_reg = -INFINITY, l_reg = 0.f;
  float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l4[4] = {0.f, 0.f, 0.f, 0.f};      // WIDE: per head of the group
  if (WIDE) for (int i = tid; i < H * H; i += nth) Tt[i] = talk ? talk[(i % H) * H + i / H] : (i % H == i / H ? 1.f : 0.f);
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
  uint32_t qf[QREG ? KS : 1][4];
  __syncthreads();
  if (QREG) {
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
      ldsm_x4(qf[QREG ? ks : 0], Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * QRS + h * DH + ks * 16 + 8 * (lane >> 4));
  }

  for (int k0 = 0; k0 < kend; k0 += TM_K) {
    cp_async_wait<0>();
    __syncthreads();                            // keys of this step have landed; everybody is done with the last step's V and P
    load_rows(Vs, k0, GD);
    cp_async_commit();
    // 1: raw scores of head h
#pragma unroll
    for (int np = 0; np < TM_K / 16; ++np) {
      float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t a[4], bk[4];
        if (QREG) { a[0] = qf[QREG ? ks : 0][0]; a[1] = qf[QREG ? ks : 0][1]; a[2] = qf[QREG ? ks : 0][2]; a[3] = qf[QREG ? ks : 0][3]; }
        else ldsm_x4(a, Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * QRS + h * DH + ks * 16 + 8 * (lane >> 4));
        ldsm_x4(bk, Ks + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * KRS + kvh * DH + ks * 16 + 8 * ((lane >> 3) & 1));
        mma_bf16(c0, a, bk[0], bk[1]);
        mma_bf16(c1, a, bk[2], bk[3]);
      }
      float* sr = S0 + (h * TM_Q + (lane >> 2)) * TM_SRS + np * 16 + 2 * (lane & 3);
      sr[0] = c0[0] * scale; sr[1] = c0[1] * scale;
      sr[8 * TM_SRS] = c0[2] * scale; sr[8 * TM_SRS + 1] = c0[3] * scale;
      sr[8] = c1[0] * scale; sr[9] = c1[1] * scale;
      sr[8 * TM_SRS + 8] = c1[2] * scale; sr[8 * TM_SRS + 9] = c1[3] * scale;
    }
    __syncthreads();                            // all raw scores are there; the key tile is free
    if (k0 + TM_K < kend) load_rows(Ks, k0 + TM_K, 0);
    cp_async_commit();
    // 2: mix, mask, online softmax
    if (WIDE) {
      const int iw = rs * RPW + (lane >> 3), kq = lane & 7;      // row, and keys [4 kq, 4 kq + 4)
      float acc[4][4];
#pragma unroll
      for (int bb = 0; bb < 4; ++bb)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[bb][j] = 0.f;
      const float* srow = S0 + iw * TM_SRS + 4 * kq;
      for (int g = 0; g < H; ++g) {
        const float4 t4 = *reinterpret_cast<const float4*>(Tt + g * H + grp * 4);
        const float tv[4] = {t4.x, t4.y, t4.z, t4.w};
        float sv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) sv[j] = srow[g * TM_Q * TM_SRS + j];
#pragma unroll
        for (int bb = 0; bb < 4; ++bb)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[bb][j] += tv[bb] * sv[j];
      }
      const int last = min(kend - 1, pos0 + iw) - (k0 + 4 * kq);
#pragma unroll
      for (int bb = 0; bb < 4; ++bb) {
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (iw >= nq || j > last) acc[bb][j] = -INFINITY;
          mx = fmaxf(mx, acc[bb][j]);
        }
#pragma unroll
        for (int mk = 1; mk < 8; mk <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, mk));
        const float mo = m4[bb], mn = fmaxf(mo, mx);
        float pj[4], sum = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) { pj[j] = mn == -INFINITY ? 0.f : __expf(acc[bb][j] - mn); sum += pj[j]; }
#pragma unroll
        for (int mk = 1; mk < 8; mk <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, mk);
        const float corr = mo == -INFINITY ? 0.f : __expf(mo - mn);
        m4[bb] = mn;
        l4[bb] = l4[bb] * corr + sum;
        const int hh = grp * 4 + bb;
        st4v(Ps + hh * PHS + iw * PRS + 4 * kq, pj[0], pj[1], pj[2], pj[3]);
        if (kq == 0) Cs[hh * TM_Q + iw] = corr;
      }
    } else if (grp * HB < H) {
      float acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = 0.f;
      const float* srow = S0 + i2 * TM_SRS + 16 * half;
#pragma unroll
      for (int g = 0; g < HP; ++g) {
        if (g < H) {
          const float tg = Tr[g];
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] += tg * srow[g * TM_Q * TM_SRS + j];
        }
      }
      const int kp0 = k0 + 16 * half;
      const int last = min(kend - 1, pos0 + i2) - kp0;          // keys 0 .. last of this half are seen
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (i2 >= nq || j > last) acc[j] = -INFINITY;
        mx = fmaxf(mx, acc[j]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float mo = m_reg, mn = fmaxf(mo, mx);
      float sum = 0.f;
      uint32_t packed[8];
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        const float p0 = mn == -INFINITY ? 0.f : __expf(acc[j] - mn), p1 = mn == -INFINITY ? 0.f : __expf(acc[j + 1] - mn);
        sum += p0 + p1;
        const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
        packed[j / 2] = *reinterpret_cast<const uint32_t*>(&pk);
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 16);
      const float corr = mo == -INFINITY ? 0.f : __expf(mo - mn);
      m_reg = mn;
      l_reg = l_reg * corr + sum;
      if (h2 < H) {
        uint32_t* pr = reinterpret_cast<uint32_t*>(Ps + h2 * PHS + i2 * PRS + 16 * half);
#pragma unroll
        for (int j = 0; j < 8; ++j) pr[j] = packed[j];
        if (half == 0) Cs[h2 * TM_Q + i2] = corr;
      }
    }
    cp_async_wait<1>();                         // the value tile (the key tile of the next step may still be in flight)
    __syncthreads();
    // 3: O_h <- O_h * corr + P_h V
    {
      const float ca = Cs[h * TM_Q + (lane >> 2)], cb = Cs[h * TM_Q + (lane >> 2) + 8];
#pragma unroll
      for (int n = 0; n < NT; ++n) { o[n][0] *= ca; o[n][1] *= ca; o[n][2] *= cb; o[n][3] *= cb; }
#pragma unroll
      for (int ks = 0; ks < TM_K / 16; ++ks) {
        uint32_t a[4];
        ldsm_x4(a, Ps + h * PHS + ((lane & 7) + 8 * ((lane >> 3) & 1)) * PRS + ks * 16 + 8 * (lane >> 4));
#pragma unroll
        for (int n2 = 0; n2 < NT / 2; ++n2) {
          uint32_t bv[4];
          ldsm_x4_t(bv, Vs + (ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * KRS + kvh * DH + n2 * 16 + 8 * (lane >> 4));
          mma_bf16(o[2 * n2], a, bv[0], bv[1]);
          mma_bf16(o[2 * n2 + 1], a, bv[2], bv[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  if (WIDE) {                                   // the statistics go to the warps that hold O
    if ((lane & 7) == 0) {
#pragma unroll
      for (int bb = 0; bb < 4; ++bb) { Cs[(grp * 4 + bb) * TM_Q + rs * RPW + (lane >> 3)] = m4[bb]; Ls[(grp * 4 + bb) * TM_Q + rs * RPW + (lane >> 3)] = l4[bb]; }
    }
  } else if (grp * HB < H && lane < TM_Q && h2 < H) {
    Cs[h2 * TM_Q + i2] = m_reg;
    Ls[h2 * TM_Q + i2] = l_reg;
  }
  __syncthreads();
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int i = (lane >> 2) + 8 * half;
    if (i < nq) {
      const float m = Cs[h * TM_Q + i];
      float l = Ls[h * TM_Q + i], e = 1.f;
      if (sink) {
        const float mm = fmaxf(m, sink[h]);
        e = expf(m - mm);
        l = l * e + expf(sink[h] - mm);
      }
      const float f = e / l * out_scale;
      bf16* dst = y + (row0 + i) * ldy + h * DH + 2 * (lane & 3);
#pragma unroll
      for (int n = 0; n < NT; ++n)
        *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) = __floats2bfloat162_rn(o[n][2 * half] * f, o[n][2 * half + 1] * f);
    }
  }
}

// one warp per (row, head): the parts' (maximum, sum, O) and the sink -> y
template <typename T>
__global__ void talk_attention_merge_kernel(const float* __restrict__ part, const float* __restrict__ sink, T* __restrict__ y, long ldy,
                                            long rows, int nparts, int H, int V, float out_scale) {
  const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= rows * H) return;
  const long row = wid / H; const int h = (int)(wid - row * H);
  const float* base = part + (row * nparts * H + h) * (long)(V + 2);
  const long step = (long)H * (V + 2);
  float M = sink ? sink[h] : -INFINITY;
  for (int s = 0; s < nparts; ++s) M = fmaxf(M, base[s * step]);
  float L = sink ? expf(sink[h] - M) : 0.f;
  for (int s = 0; s < nparts; ++s) { const float m = base[s * step]; if (m != -INFINITY) L += base[s * step + 1] * expf(m - M); }
  for (int v = lane; v < V; v += 32) {
    float o = 0.f;
    for (int s = 0; s < nparts; ++s) { const float m = base[s * step]; if (m != -INFINITY) o += base[s * step + 2 + v] * expf(m - M); }
    stf(y + row * ldy + h * V + v, o / L * out_scale);
  }
}

}  // namespace

// ====================================================================================================================
// launchers (C ABI; return 0, a CUDA error code, or -1 for sizes a kernel is not built for)
// ====================================================================================================================
#define LAUNCH_END() do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : (int)e_; } while (0)

extern "C" {

int lbp_postnorm_residual(const float* xin, float* xout, const void* y1, long ldy1, int y1dtype, const float* y2, long ldy2,
                          const int* pos, const float* cw, int top, float alpha, const void* w, float eps, void* h, long ldh,
                          long rows, int n, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  const size_t smem = (size_t)n * sizeof(float);
  if (smem > 160 * 1024) return -1;
  const int esz = dtype ? 2 : 4, y1sz = y1dtype ? 2 : 4;
  const bool vec = n % 4 == 0 && ((uintptr_t)xin & 15) == 0 && ((uintptr_t)xout & 15) == 0 && ((uintptr_t)w % (4 * esz)) == 0 &&
                   (!y1 || (((uintptr_t)y1 % (4 * y1sz)) == 0 && ldy1 % 4 == 0)) && (!y2 || (((uintptr_t)y2 & 15) == 0 && ldy2 % 4 == 0)) &&
                   (!h || (((uintptr_t)h % (4 * esz)) == 0 && ldh % 4 == 0));
  if (vec && n / 4 <= 2048) {                   // the row in registers: one or two quadruples per thread
    const int quads = n / 4, items = quads <= 256 ? 1 : 2;
    int vthreads = (((quads + items - 1) / items + 31) / 32) * 32;
    if (vthreads > 1024) vthreads = 1024;
#define PNV(TT, TY, IT) postnorm_residual_vec_kernel<TT, TY, IT><<<(unsigned)rows, vthreads, 0, s>>>(xin, xout, (const TY*)y1, ldy1, y2, ldy2, pos, cw, top, \
        alpha, (const TT*)w, eps, (TT*)h, ldh, n)
#define PNV2(TT, TY) { if (items == 1) PNV(TT, TY, 1); else PNV(TT, TY, 2); }
    if (dtype) { if (y1dtype) PNV2(bf16, bf16) else PNV2(bf16, float) }
    else { if (y1dtype) return -1; PNV2(float, float) }
#undef PNV2
#undef PNV
    LAUNCH_END();
  }
  const int threads = n >= 2048 ? 256 : 128;
#define PN(TT, TY) { \
    if (smem > 48 * 1024) cudaFuncSetAttribute(postnorm_residual_kernel<TT, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    postnorm_residual_kernel<TT, TY><<<(unsigned)rows, threads, smem, s>>>(xin, xout, (const TY*)y1, ldy1, y2, ldy2, pos, cw, top, alpha, \
                                                                           (const TT*)w, eps, (TT*)h, ldh, n); }
  if (dtype) { if (y1dtype) PN(bf16, bf16) else PN(bf16, float) }
  else { if (y1dtype) return -1; PN(float, float) }
#undef PN
  LAUNCH_END();
}

int lbp_conv_qkv_prepare(const void* qin, const void* kin, const void* vin, long ld, const void* wq, const void* wk, const void* wv,
                         int taps, void* tail, const void* qn, const void* kn, const float* freq, int half, float eps, void* qout,
                         long ldqo, void* pool, const int* table, int max_pages, int page_size, const int* tok_seq,
                         const int* seq_off, const int* slots, const int* past, long tokens, int B, int H, int G, int D, int V,
                         int dtype, cudaStream_t s) {
  if (tokens == 0) return 0;
  if (taps < 1 || 2 * half > D) return -1;
  const int W = D > V ? D : V, warps = 4;
  const size_t smem = (size_t)warps * W * sizeof(float);
  if (smem > 48 * 1024) return -1;
  const long units = tokens * (H + 2 * G);
  const unsigned grid = (unsigned)((units + warps - 1) / warps);
  const int C = H * D + G * D + G * V;
  const int esz = dtype ? 2 : 4;
  const bool v4 = D % 4 == 0 && V % 4 == 0 && ld % 4 == 0 && ((uintptr_t)qin % (4 * esz)) == 0 && ((uintptr_t)kin % (4 * esz)) == 0 &&
                  ((uintptr_t)vin % (4 * esz)) == 0 && ((uintptr_t)tail % (4 * esz)) == 0;
#define CQ(TT, VV) conv_qkv_prepare_kernel<TT, VV><<<grid, warps * 32, smem, s>>>((const TT*)qin, (const TT*)kin, (const TT*)vin, ld, (const TT*)wq, \
        (const TT*)wk, (const TT*)wv, taps, (const TT*)tail, (const TT*)qn, (const TT*)kn, freq, half, eps, (TT*)qout, ldqo, (TT*)pool, table, \
        max_pages, page_size, tok_seq, seq_off, slots, past, tokens, H, G, D, V, W)
  if (dtype) { if (v4) CQ(bf16, 4); else CQ(bf16, 1); } else { if (v4) CQ(float, 4); else CQ(float, 1); }
#undef CQ
  if (taps > 1) {
    const dim3 tg((C + 127) / 128, B);
    if (dtype) conv_tail_update_kernel<bf16><<<tg, 128, 0, s>>>((const bf16*)qin, (const bf16*)kin, (const bf16*)vin, ld, (bf16*)tail, taps - 1,
                                                               seq_off, slots, past, H * D, G * D, G * V);
    else conv_tail_update_kernel<float><<<tg, 128, 0, s>>>((const float*)qin, (const float*)kin, (const float*)vin, ld, (float*)tail, taps - 1,
                                                            seq_off, slots, past, H * D, G * D, G * V);
  }
  LAUNCH_END();
}

// shared memory of one attention block, in floats
static size_t talk_smem_floats(int QT, int KT, int H, int G, int D, int V) {
  return (size_t)QT * H * D + (size_t)QT * H * V + (size_t)KT * (G * D + 1) + (size_t)KT * G * V + 2 * (size_t)H * QT * KT +
         3 * (size_t)H * QT + (size_t)H * H;
}

// the largest query tile (at most qt_max) and key tile that fit the block's shared memory; 0 when nothing fits
int lbp_talk_attention_tiles(int qt_max, int H, int G, int D, int V, int* kt_out) {
  const size_t cap = 200 * 1024 / sizeof(float);
  for (int kt = 32; kt >= 1; kt >>= 1) {
    for (int qt = qt_max; qt >= 1; qt >>= 1) {
      if (kt < 32 && qt > 2) continue;          // a short key tile only where even two queries do not fit a long one
      if (talk_smem_floats(qt, kt, H, G, D, V) <= cap) { *kt_out = kt; return qt; }
    }
  }
  return 0;
}

int lbp_talk_attention(const void* q, long ldq, const void* pool, const int* table, int max_pages, int page_size, const float* talk,
                       const float* sink, const int* qt_seq, const int* qt_start, int ntiles, int QT, int KT, const int* seq_off,
                       const int* slots, const int* past, void* y, long ldy, float* part, int nparts, long rows, int H, int G, int D,
                       int V, float scale, float out_scale, int dtype, cudaStream_t s) {
  if (ntiles == 0) return 0;
  if (H % G != 0 || nparts < 1 || (nparts > 1 && !part)) return -1;
  const size_t smem = talk_smem_floats(QT, KT, H, G, D, V) * sizeof(float);
  if (smem > 200 * 1024) return -1;
  const dim3 grid((unsigned)ntiles, (unsigned)nparts);
#define TA(TT, Q) { \
    if (smem > 48 * 1024) cudaFuncSetAttribute(talk_attention_kernel<TT, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    talk_attention_kernel<TT, Q><<<grid, 256, smem, s>>>((const TT*)q, ldq, (const TT*)pool, table, max_pages, page_size, talk, sink, qt_seq, \
        qt_start, seq_off, slots, past, (TT*)y, ldy, part, nparts, KT, H, G, D, V, scale, out_scale); }
#define TAQ(TT) { if (QT == 1) TA(TT, 1) else if (QT == 2) TA(TT, 2) else if (QT == 4) TA(TT, 4) else if (QT == 8) TA(TT, 8) else return -1; }
  if (dtype) TAQ(bf16) else TAQ(float)
#undef TAQ
#undef TA
  if (nparts > 1) {
    const unsigned mg = (unsigned)((rows * H * 32 + 255) / 256);
    if (dtype) talk_attention_merge_kernel<bf16><<<mg, 256, 0, s>>>(part, sink, (bf16*)y, ldy, rows, nparts, H, V, out_scale);
    else talk_attention_merge_kernel<float><<<mg, 256, 0, s>>>(part, sink, (float*)y, ldy, rows, nparts, H, V, out_scale);
  }
  LAUNCH_END();
}

// tensor-core prompt kernel: bf16, equal key and value head sizes of 64 or 128, at most 16 heads; -1 otherwise
int lbp_talk_attention_mma(const void* q, long ldq, const void* pool, const int* table, int max_pages, int page_size, const float* talk,
                           const float* sink, const int* qt_seq, const int* qt_start, int ntiles, const int* seq_off, const int* slots,
                           const int* past, void* y, long ldy, int H, int G, int D, int V, float scale, float out_scale, cudaStream_t s) {
  if (ntiles == 0) return 0;
  if (D != V || (D != 64 && D != 128) || H < 1 || H > 16 || H % G != 0 || ldq % 8 != 0 || ldy % 2 != 0 || (H * 32) % (G * D / 8) != 0 ||
      ((uintptr_t)q & 15) != 0 || ((uintptr_t)pool & 15) != 0 || ((uintptr_t)y & 3) != 0) return -1;
  const int hp = H <= 8 ? 8 : 16;
  const int hb = H % 4 == 0 ? 4 : ((hp == 16 && H % 2 == 0) ? 2 : 1);
  const int GD = G * D;
  const size_t smem = (size_t)2 * (2 * TM_K * (GD + 8) + TM_Q * (H * D + 8) + H * TM_PHS) + (size_t)4 * (H * TM_Q * TM_SRS + 2 * H * TM_Q + H * H);
  if (smem > 220 * 1024) return -1;
#define TM(DH_, HP_, HB_, QR_) { \
    cudaFuncSetAttribute(talk_attention_mma_kernel<DH_, HP_, HB_, QR_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    talk_attention_mma_kernel<DH_, HP_, HB_, QR_><<<(unsigned)ntiles, H * 32, smem, s>>>((const bf16*)q, ldq, (const bf16*)pool, table, max_pages, \
        page_size, talk, sink, qt_seq, qt_start, seq_off, slots, past, (bf16*)y, ldy, H, G, scale, out_scale); }
  if (D == 64) {
    if (hp == 8) { if (hb == 4) TM(64, 8, 4, true) else TM(64, 8, 1, true) }
    else { if (hb == 4) TM(64, 16, 4, false) else if (hb == 2) TM(64, 16, 2, false) else TM(64, 16, 1, false) }
  } else {
    if (hp == 8) { if (hb == 4) TM(128, 8, 4, true) else TM(128, 8, 1, true) }
    else { if (hb == 4) TM(128, 16, 4, false) else if (hb == 2) TM(128, 16, 2, false) else TM(128, 16, 1, false) }
  }
#undef TM
  LAUNCH_END();
}

}  // extern "C"
