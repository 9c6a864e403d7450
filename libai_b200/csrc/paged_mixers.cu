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
template <typename T>
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
  for (int c = lane; c < n; c += 32) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int lt = t - R + j;
      float uv = 0.f;
      if (lt >= 0) uv = ldf(in + (long)(s0 + lt) * ld + c);
      else if (pb + lt >= 0) uv = ldf(tail + ((long)slot * R + (R + lt)) * C + coff + c);
      acc += ldf(cw + (long)c * taps + j) * uv;
    }
    buf[c] = acc;
    ss += acc * acc;
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)n + eps);
  __syncwarp();
  T* krow = pool + ((long)table[(long)slot * max_pages + p / page_size] * page_size + p % page_size) * (long)(G * D + G * V);
  if (kind == 2) {
    for (int c = lane; c < n; c += 32) stf(krow + G * D + hh * V + c, buf[c] * r);
    return;
  }
  const T* nw = kind == 0 ? qn : kn;
  T* dst = kind == 0 ? qout + tok * ldqo + hh * D : krow + hh * D;
  for (int c = lane; c < n; c += 32) {
    float o = buf[c] * r * ldf(nw + c);
    if (c < 2 * half) {
      const int i = c < half ? c : c - half;
      const float ang = (float)p * freq[i];
      const float cs = cosf(ang), sn = sinf(ang);
      if (c < half) o = o * cs - buf[c + half] * r * ldf(nw + c + half) * sn;
      else o = o * cs + buf[c - half] * r * ldf(nw + c - half) * sn;
    }
    stf(dst + c, o);
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
  const int b = qt_seq[blockIdx.x], t0 = qt_start[blockIdx.x];
  const int s0 = seq_off[b], nq = min(QT, seq_off[b + 1] - s0 - t0), pos0 = past[b] + t0;
  const long row0 = s0 + t0;
  const long slot = slots[b];
  const int kall = pos0 + nq;                                   // keys the tile's last query sees
  int len = (kall + nparts - 1) / nparts;
  len = (len + KT - 1) / KT * KT;
  const int kbeg = blockIdx.y * len, kend = min(kall, kbeg + len);
  const long C = GD + GV;

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
        for (int c = lane; c < GD; c += 32) Ks[j * KP + c] = ldf(rowp + c);
        for (int c = lane; c < GV; c += 32) Vs[j * GV + c] = ldf(rowp + GD + c);
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
//   2  the mix over heads on the fp32 pipe: warp w takes HB output heads and 16 / HB of the rows, lane = key, the rows of
//      `talk` of its heads in registers, so that a loaded raw score feeds HB multiply-adds; causal mask; online softmax (the
//      running maximum and sum of the warp's 16 (head, row) pairs live in lanes 0..15); probabilities as bf16 and the
//      correction factors into shared memory;
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

constexpr int TM_Q = 16, TM_K = 32, TM_SRS = TM_K + 8;           // queries, keys per tile; row stride of the fp32 scores

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
  constexpr int PRS = TM_K + 8;
  bf16* Ks = reinterpret_cast<bf16*>(smraw);
  bf16* Vs = Ks + TM_K * KRS;
  bf16* Qs = Vs + TM_K * KRS;
  bf16* Ps = Qs + TM_Q * QRS;                   // [H][16][PRS]
  float* S0 = reinterpret_cast<float*>(Ps + H * TM_Q * PRS);   // [H][16][TM_SRS]
  float* Cs = S0 + H * TM_Q * TM_SRS;           // [H][16] correction of this tile, then the final maximum
  float* Ls = Cs + H * TM_Q;                    // [H][16] final sum
  const int tid = threadIdx.x, nth = blockDim.x, warp = tid >> 5, lane = tid & 31;
  const int b = qt_seq[blockIdx.x], t0 = qt_start[blockIdx.x];
  const int s0 = seq_off[b], nq = min(TM_Q, seq_off[b + 1] - s0 - t0), pos0 = past[b] + t0;
  const long row0 = s0 + t0;
  const long slot = slots[b];
  const int kend = pos0 + nq;
  const int h = warp, kvh = h / rep;

  auto load_rows = [&](bf16* dst, int k0, int coff) {            // 32 cache rows, columns [coff, coff + GD), 16 bytes per copy
    const int per = GD / 8;
    for (int i = tid; i < TM_K * per; i += nth) {
      const int j = i / per, c = (i - j * per) * 8;
      const int kp = k0 + j;
      if (kp < kend) {
        const bf16* rowp = pool + ((long)table[slot * max_pages + kp / page_size] * page_size + kp % page_size) * (long)C + coff;
        cp_async16(dst + j * KRS + c, rowp + c);
      } else {
        *reinterpret_cast<uint4*>(dst + j * KRS + c) = make_uint4(0u, 0u, 0u, 0u);
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
  // phase-2 role of this warp: heads grp * HB .. + HB - 1, rows rs * RPW .. + RPW - 1; lane r < 16 keeps the statistics of
  // (head grp * HB + r / RPW, row rs * RPW + r % RPW)
  const int grp = warp / HB, rs = warp % HB;
  float Tr[HB][HP];
#pragma unroll
  for (int bb = 0; bb < HB; ++bb)
#pragma unroll
    for (int g = 0; g < HP; ++g) {
      const int hh = grp * HB + bb;
      Tr[bb][g] = (g < H && hh < H) ? (talk ? talk[hh * H + g] : (g == hh ? 1.f : 0.f)) : 0.f;
    }
  float m_reg = -INFINITY, l_reg = 0.f;
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
      *reinterpret_cast<float2*>(sr) = make_float2(c0[0] * scale, c0[1] * scale);
      *reinterpret_cast<float2*>(sr + 8 * TM_SRS) = make_float2(c0[2] * scale, c0[3] * scale);
      *reinterpret_cast<float2*>(sr + 8) = make_float2(c1[0] * scale, c1[1] * scale);
      *reinterpret_cast<float2*>(sr + 8 * TM_SRS + 8) = make_float2(c1[2] * scale, c1[3] * scale);
    }
    __syncthreads();                            // all raw scores are there; the key tile is free
    if (k0 + TM_K < kend) load_rows(Ks, k0 + TM_K, 0);
    cp_async_commit();
    // 2: mix, mask, online softmax
    if (grp * HB < H) {
      const int kp = k0 + lane;
      for (int rl = 0; rl < RPW; ++rl) {
        const int i = rs * RPW + rl;
        float acc[HB];
#pragma unroll
        for (int bb = 0; bb < HB; ++bb) acc[bb] = 0.f;
#pragma unroll
        for (int g = 0; g < HP; ++g) {
          if (g < H) {
            const float sv = S0[(g * TM_Q + i) * TM_SRS + lane];
#pragma unroll
            for (int bb = 0; bb < HB; ++bb) acc[bb] += Tr[bb][g] * sv;
          }
        }
        const bool seen = i < nq && kp < kend && kp <= pos0 + i;
#pragma unroll
        for (int bb = 0; bb < HB; ++bb) {
          const int hh = grp * HB + bb, r = bb * RPW + rl;
          const float v = seen ? acc[bb] : -INFINITY;
          const float mx = warp_max(v);
          const float mo = __shfl_sync(0xffffffffu, m_reg, r);
          const float mn = fmaxf(mo, mx);
          const float pj = mn == -INFINITY ? 0.f : expf(v - mn);
          const float sum = warp_sum(pj);
          const float corr = mo == -INFINITY ? 0.f : expf(mo - mn);
          if (lane == r) { m_reg = mn; l_reg = l_reg * corr + sum; }
          if (hh < H) {
            Ps[(hh * TM_Q + i) * PRS + lane] = __float2bfloat16_rn(pj);
            if (lane == 0) Cs[hh * TM_Q + i] = corr;
          }
        }
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
        ldsm_x4(a, Ps + (h * TM_Q + (lane & 7) + 8 * ((lane >> 3) & 1)) * PRS + ks * 16 + 8 * (lane >> 4));
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
  if (grp * HB < H && lane < TM_Q) {            // the statistics go to the warps that hold O
    const int hh = grp * HB + lane / RPW, i = rs * RPW + lane % RPW;
    if (hh < H) { Cs[hh * TM_Q + i] = m_reg; Ls[hh * TM_Q + i] = l_reg; }
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
  if (dtype) {
    conv_qkv_prepare_kernel<bf16><<<grid, warps * 32, smem, s>>>((const bf16*)qin, (const bf16*)kin, (const bf16*)vin, ld, (const bf16*)wq,
        (const bf16*)wk, (const bf16*)wv, taps, (const bf16*)tail, (const bf16*)qn, (const bf16*)kn, freq, half, eps, (bf16*)qout, ldqo,
        (bf16*)pool, table, max_pages, page_size, tok_seq, seq_off, slots, past, tokens, H, G, D, V, W);
    if (taps > 1) conv_tail_update_kernel<bf16><<<dim3((C + 127) / 128, B), 128, 0, s>>>((const bf16*)qin, (const bf16*)kin, (const bf16*)vin,
        ld, (bf16*)tail, taps - 1, seq_off, slots, past, H * D, G * D, G * V);
  } else {
    conv_qkv_prepare_kernel<float><<<grid, warps * 32, smem, s>>>((const float*)qin, (const float*)kin, (const float*)vin, ld,
        (const float*)wq, (const float*)wk, (const float*)wv, taps, (const float*)tail, (const float*)qn, (const float*)kn, freq, half,
        eps, (float*)qout, ldqo, (float*)pool, table, max_pages, page_size, tok_seq, seq_off, slots, past, tokens, H, G, D, V, W);
    if (taps > 1) conv_tail_update_kernel<float><<<dim3((C + 127) / 128, B), 128, 0, s>>>((const float*)qin, (const float*)kin,
        (const float*)vin, ld, (float*)tail, taps - 1, seq_off, slots, past, H * D, G * D, G * V);
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
  for (int kt = 32; kt >= 8; kt >>= 1) {
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
  if (D != V || (D != 64 && D != 128) || H < 1 || H > 16 || H % G != 0 || ldq % 8 != 0 || ldy % 2 != 0 ||
      ((uintptr_t)q & 15) != 0 || ((uintptr_t)pool & 15) != 0 || ((uintptr_t)y & 3) != 0) return -1;
  const int hp = H <= 8 ? 8 : 16;
  const int hb = (hp == 8 && H % 4 == 0) ? 4 : ((hp == 16 && H % 2 == 0) ? 2 : 1);
  const int GD = G * D;
  const size_t smem = (size_t)2 * (2 * TM_K * (GD + 8) + TM_Q * (H * D + 8) + H * TM_Q * (TM_K + 8)) +
                      (size_t)4 * (H * TM_Q * TM_SRS + 2 * H * TM_Q);
  if (smem > 220 * 1024) return -1;
#define TM(DH_, HP_, HB_, QR_) { \
    cudaFuncSetAttribute(talk_attention_mma_kernel<DH_, HP_, HB_, QR_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    talk_attention_mma_kernel<DH_, HP_, HB_, QR_><<<(unsigned)ntiles, H * 32, smem, s>>>((const bf16*)q, ldq, (const bf16*)pool, table, max_pages, \
        page_size, talk, sink, qt_seq, qt_start, seq_off, slots, past, (bf16*)y, ldy, H, G, scale, out_scale); }
  if (D == 64) {
    if (hp == 8) { if (hb == 4) TM(64, 8, 4, true) else TM(64, 8, 1, true) }
    else { if (hb == 2) TM(64, 16, 2, false) else TM(64, 16, 1, false) }
  } else {
    if (hp == 8) { if (hb == 4) TM(128, 8, 4, true) else TM(128, 8, 1, true) }
    else { if (hb == 2) TM(128, 16, 2, false) else TM(128, 16, 1, false) }
  }
#undef TM
  LAUNCH_END();
}

}  // extern "C"
