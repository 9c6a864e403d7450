// Kernels of decoders whose sequence mixers are linear-attention recurrences with a decay, on several residual streams:
// token + bigram embedding, hyper-connection streams fused with the RMS norm that opens the next sublayer, the decayed
// outer-product recurrence (one fixed decay per head, or one data-dependent decay per key channel) with its fp32 state,
// and the gated RMS norm of the read-out.
//
// Conventions (the same ragged-batch descriptor as seq_mixers.cu / kv_mixers.cu).  A step carries B sequences; sequence
// b brings n_b = seq_off[b+1]-seq_off[b] new tokens packed at rows seq_off[b].. of every activation matrix, has past[b]
// tokens already folded into its state, which lives in slot slots[b]; a sequence with past[b] == 0 never reads its slot.
// Activations are `T` (float or bf16, `dtype` 0 / 1); the residual streams, norms, decays and the recurrence are fp32
// in both.  Built WITHOUT fast-math: the fp32 mode is exact to rounding.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace {

using bf16 = __nv_bfloat16;

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// four consecutive channels (16-byte fp32 / 8-byte bf16 accesses)
template <typename T> __device__ __forceinline__ float4 ld4(const T* p);
template <> __device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld4<bf16>(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename T> __device__ __forceinline__ void st4(T* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<bf16>(bf16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&a); raw.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}
// sum over the block (blockDim.x a multiple of 32, at most 1024); every thread gets the result
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
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
// log(sigmoid(x)) without cancellation: min(x, 0) - log1p(exp(-|x|))
__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// ------------------------------------------------------------------------------------------------------------------
// Embedding: x[r] = table[ids[r]] * scale + bigram[row(r)], written to every one of `ns` residual streams
// (x: [ns, rows, n] fp32).  row(r) = (previous token * mul_prev + token * mul_cur) mod buckets; the first token of a
// sequence takes row `buckets`.  The previous token of a step's first row is last[slot] (the sequence's state) when
// past > 0.  token_last_kernel then stores every sequence's last token of the step (a second launch: the first rows of
// the step must have read `last` before it changes).
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_bigram_kernel(const T* __restrict__ table, const T* __restrict__ bigram, const int64_t* __restrict__ ids,
                                    const int* __restrict__ last, const int* __restrict__ tok_seq, const int* __restrict__ seq_off,
                                    const int* __restrict__ slots, const int* __restrict__ past, float scale, long mul_prev,
                                    long mul_cur, long buckets, float* __restrict__ x, long rows, int n, int ns, int vec) {
  const long r = blockIdx.x;
  const int b = tok_seq[r];
  const long tok = ids[r];
  long prev = -1;
  if (r > seq_off[b]) prev = ids[r - 1];
  else if (past[b] > 0) prev = last[slots[b]];
  const long row = prev < 0 ? buckets : (prev * mul_prev + tok * mul_cur) % buckets;
  const T* e = table + tok * n;
  const T* g = bigram + row * n;
  if (vec) {
    for (int c = threadIdx.x * 4; c < n; c += blockDim.x * 4) {
      const float4 a = ld4(e + c), d = ld4(g + c);
      const float4 v = make_float4(a.x * scale + d.x, a.y * scale + d.y, a.z * scale + d.z, a.w * scale + d.w);
      for (int s = 0; s < ns; ++s) *reinterpret_cast<float4*>(x + ((long)s * rows + r) * n + c) = v;
    }
  } else {
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      const float v = ldf(e + c) * scale + ldf(g + c);
      for (int s = 0; s < ns; ++s) x[((long)s * rows + r) * n + c] = v;
    }
  }
}

__global__ void token_last_kernel(const int64_t* __restrict__ ids, int* __restrict__ last, const int* __restrict__ seq_off,
                                  const int* __restrict__ slots, int B) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) last[slots[b]] = (int)ids[seq_off[b + 1] - 1];
}

// ------------------------------------------------------------------------------------------------------------------
// Hyper-connections: `ns` residual streams x_1..x_ns ([ns, rows, n] fp32, updated in place).  One block per row:
//   closing a sublayer (y given):   x_t <- sum_s mix[s, t] x_s + out[t] * y     (all t from the old streams; y: rows of
//                                   the sublayer's output, or - `pos` given - sum_k cw[r,k] * y[pos[r,k]] over sorted
//                                   expert rows)
//   opening the next (h given):     u = sum_s inw[s] x_s;  h = u / sqrt(mean(u^2) + eps) * w
// mix / out / inw are fp32.  This is the general form (any width and alignment, up to HC_MAXS streams): one channel per thread
// and access, u kept in shared memory between the two passes over the row.
// ------------------------------------------------------------------------------------------------------------------
constexpr int HC_MAXS = 16;

template <typename T, typename Ty>
__global__ void hc_step_kernel(float* __restrict__ x, long rows, int n, int ns, const Ty* __restrict__ y, long ldy,
                               const int* __restrict__ pos, const float* __restrict__ cw, int top, const float* __restrict__ mix,
                               const float* __restrict__ outw, const float* __restrict__ inw, const T* __restrict__ w, float eps,
                               T* __restrict__ h, long ldh) {
  extern __shared__ __align__(16) float hc_sm[];
  float* u = hc_sm;                                  // [n] (only with h)
  __shared__ float coef[HC_MAXS * HC_MAXS + 2 * HC_MAXS];
  __shared__ float red[32];
  const long r = blockIdx.x;
  for (int i = threadIdx.x; i < ns * ns; i += blockDim.x) coef[i] = y ? mix[i] : 0.f;
  if (threadIdx.x < ns) {
    coef[HC_MAXS * HC_MAXS + threadIdx.x] = y ? outw[threadIdx.x] : 0.f;
    coef[HC_MAXS * HC_MAXS + HC_MAXS + threadIdx.x] = h ? inw[threadIdx.x] : 0.f;
  }
  __syncthreads();
  const float* cm = coef;
  const float* co = coef + HC_MAXS * HC_MAXS;
  const float* ci = co + HC_MAXS;
  float ss = 0.f;
  {
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      float xs[HC_MAXS];
#pragma unroll
      for (int s = 0; s < HC_MAXS; ++s) if (s < ns) xs[s] = x[((long)s * rows + r) * n + c];
      if (y) {
        float yv = 0.f;
        if (pos) { for (int k = 0; k < top; ++k) yv += cw[r * top + k] * ldf(y + (long)pos[r * top + k] * ldy + c); }
        else yv = ldf(y + r * ldy + c);
        float nx[HC_MAXS];
#pragma unroll
        for (int t = 0; t < HC_MAXS; ++t) {
          if (t < ns) {
            float a = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAXS; ++s) if (s < ns) a += cm[s * ns + t] * xs[s];
            nx[t] = a + co[t] * yv;
          }
        }
#pragma unroll
        for (int t = 0; t < HC_MAXS; ++t) if (t < ns) { xs[t] = nx[t]; x[((long)t * rows + r) * n + c] = nx[t]; }
      }
      if (h) {
        float uv = 0.f;
#pragma unroll
        for (int s = 0; s < HC_MAXS; ++s) if (s < ns) uv += ci[s] * xs[s];
        u[c] = uv;
        ss += uv * uv;
      }
    }
  }
  if (!h) return;
  ss = block_sum(ss, red);
  const float rr = 1.f / sqrtf(ss / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x) stf(h + r * ldh + c, u[c] * rr * ldf(w + c));
}

// The same for rows of 16-byte aligned fp32 quadruples with at most NS streams and ITEMS quadruples per thread: every load of
// the row is issued before the first store (the streams are read and written through one pointer, so the compiler keeps the
// program order of a load that follows a store), and u stays in registers between the two passes.
template <typename T, typename Ty, int NS, int ITEMS>
__global__ void hc_step_vec_kernel(float* __restrict__ x, long rows, int n, int ns, const Ty* __restrict__ y, long ldy,
                                   const int* __restrict__ pos, const float* __restrict__ cw, int top, const float* __restrict__ mix,
                                   const float* __restrict__ outw, const float* __restrict__ inw, const T* __restrict__ w, float eps,
                                   T* __restrict__ h, long ldh) {
  __shared__ float red[32];
  const long r = blockIdx.x;
  float cm[NS][NS], co[NS], ci[NS];
#pragma unroll
  for (int a = 0; a < NS; ++a) {
    co[a] = (y && a < ns) ? outw[a] : 0.f;
    ci[a] = (h && a < ns) ? inw[a] : 0.f;
#pragma unroll
    for (int b = 0; b < NS; ++b) cm[a][b] = (y && a < ns && b < ns) ? mix[a * ns + b] : 0.f;
  }
  float4 xs[ITEMS][NS], yv[ITEMS], uv[ITEMS];
  int col[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    col[i] = (threadIdx.x + i * blockDim.x) * 4;
    const bool ok = col[i] < n;
#pragma unroll
    for (int a = 0; a < NS; ++a)
      xs[i][a] = (ok && a < ns) ? *reinterpret_cast<const float4*>(x + ((long)a * rows + r) * n + col[i]) : make_float4(0.f, 0.f, 0.f, 0.f);
    yv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (y && ok) {
      if (pos) {
        for (int k = 0; k < top; ++k) {
          const float wk = cw[r * top + k];
          const float4 t = ld4(y + (long)pos[r * top + k] * ldy + col[i]);
          yv[i].x += wk * t.x; yv[i].y += wk * t.y; yv[i].z += wk * t.z; yv[i].w += wk * t.w;
        }
      } else {
        yv[i] = ld4(y + r * ldy + col[i]);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const bool ok = col[i] < n;
    if (y) {
      float4 nx[NS];
#pragma unroll
      for (int t = 0; t < NS; ++t) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int q = 0; q < NS; ++q) {            // in the order of the general kernel: streams first, then the output
          const float m = cm[q][t];
          a.x += m * xs[i][q].x; a.y += m * xs[i][q].y; a.z += m * xs[i][q].z; a.w += m * xs[i][q].w;
        }
        a.x += co[t] * yv[i].x; a.y += co[t] * yv[i].y; a.z += co[t] * yv[i].z; a.w += co[t] * yv[i].w;
        nx[t] = a;
      }
#pragma unroll
      for (int t = 0; t < NS; ++t) {
        xs[i][t] = nx[t];
        if (ok && t < ns) *reinterpret_cast<float4*>(x + ((long)t * rows + r) * n + col[i]) = nx[t];
      }
    }
    float4 u4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < NS; ++q) { u4.x += ci[q] * xs[i][q].x; u4.y += ci[q] * xs[i][q].y; u4.z += ci[q] * xs[i][q].z; u4.w += ci[q] * xs[i][q].w; }
    uv[i] = u4;
    ss += u4.x * u4.x + u4.y * u4.y + u4.z * u4.z + u4.w * u4.w;
  }
  if (!h) return;
  ss = block_sum(ss, red);
  const float rr = 1.f / sqrtf(ss / (float)n + eps);
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    if (col[i] < n) {
      const float4 wv = ld4(w + col[i]);
      st4(h + r * ldh + col[i], make_float4(uv[i].x * rr * wv.x, uv[i].y * rr * wv.y, uv[i].z * rr * wv.z, uv[i].w * rr * wv.w));
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Decayed outer-product recurrence (linear attention).  Per head, with S [D, V] in fp32:
//   S <- diag(a_t) S + k_t v_t^T;   o_t = S^T q_t
// a_t is one fixed number per head (`decay` [H], `z` absent) or one per key channel and token,
// a = sigmoid(z + zb)^(inv_tau) = exp(inv_tau * log sigmoid(z + zb)) with the logits z [tokens, H*D] in fp32.
// With `lower` [H*D] the decay is bounded from below and also decides what is written (the forget gate of HGRN2):
//   a = lower + (1 - lower) * sigmoid(z + zb),   k = 1 - a   (the k argument is not read).
// q, k, v are column slices of the projection output (row stride ld*); `act` is a bit mask of the ones that pass through
// SiLU (1: q, 2: k, 4: v); q is multiplied by q_scale and k by k_scale (fp32).
//
// Columns of S are independent: a block owns `VT` of them for one (sequence, head).  A thread keeps a DPT x 8 tile of S
// in registers: DPT consecutive key rows (lane r of the R = ceil(D/DPT) adjacent lanes that share a column group) of 8
// consecutive columns, so the 2*DPT k and q numbers and 8 values a thread fetches from shared memory per token feed
// 24*DPT fused multiply-adds: the arithmetic, not the shared-memory traffic, is the bound (a thread per column re-reads
// k and q for every column).  The eight partial read-outs are summed over the R lanes by a transposing butterfly
// (8 shuffles for R = 16).  Tokens are staged through shared memory CT (at most SCAN_CT) at a time as fp32 (rows of lane r at
// a padded offset: 16-byte loads without bank conflicts) with activations, scales and decays applied during staging; the
// global loads of the next group are issued before the serial walk over the current one and land in the other buffer
// afterwards.
// ------------------------------------------------------------------------------------------------------------------
constexpr int SCAN_CT = 16, SCAN_NC = 8;

template <typename T, int N> __device__ __forceinline__ void ldn(const T* p, float (&f)[N]);
template <> __device__ __forceinline__ void ldn<float, 4>(const float* p, float (&f)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
}
template <> __device__ __forceinline__ void ldn<float, 8>(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <> __device__ __forceinline__ void ldn<bf16, 4>(const bf16* p, float (&f)[4]) {
  const float4 a = ld4(p);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
}
template <> __device__ __forceinline__ void ldn<bf16, 8>(const bf16* p, float (&f)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(h2[i]); f[2 * i + 1] = __high2float(h2[i]); }
}

template <typename T, int DPT>
__global__ void __launch_bounds__(256, 1)
decay_scan_kernel(const T* __restrict__ q, long ldq, const T* __restrict__ k, long ldk, const T* __restrict__ v, long ldv,
                  const float* __restrict__ decay, const float* __restrict__ z, long ldz, const float* __restrict__ zb,
                  const float* __restrict__ lower, float inv_tau, float q_scale, float k_scale, int act, float* __restrict__ S, const int* __restrict__ seq_off,
                  const int* __restrict__ slots, const int* __restrict__ past, float* __restrict__ out, int H, int D, int V, int R,
                  int VT, int CT, int vec) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NC = SCAN_NC, PS = DPT == 8 ? 12 : 4;   // padded stride of one lane's rows
  const int b = blockIdx.x / H, h = blockIdx.x % H;
  const int j0 = blockIdx.y * VT;
  const int Dp = R * PS;                        // floats per staged token
  const bool chan = z != nullptr;
  const int buf_floats = CT * (Dp * (chan ? 3 : 2) + VT);
  const int tid = threadIdx.x, nth = blockDim.x;
  const int r = tid % R, grp = tid / R;         // lane within the column group, column group
  const int jc = j0 + grp * NC;                 // first of this thread's 8 columns
  const bool grp_ok = grp * NC < VT;
  const int n = seq_off[b + 1] - seq_off[b];
  const long tok0 = seq_off[b];
  const float g0 = chan ? 1.f : decay[h];
  float* Sg = S + ((long)slots[b] * H + h) * (long)D * V;
  float s[DPT][NC];
#pragma unroll
  for (int d = 0; d < DPT; ++d) {
    const int i = r * DPT + d;
#pragma unroll
    for (int c = 0; c < NC; ++c) s[d][c] = (past[b] > 0 && grp_ok && i < D && jc + c < V) ? Sg[(long)i * V + jc + c] : 0.f;
  }
  // staging work of this thread: one (token, lane chunk) of q / k / decays and one (token, column group) of v per group of CT
  // tokens (the launcher picks CT so that both fit the block)
  const int qk_items = CT * R, v_items = CT * (VT / NC);
  float rk[DPT], rq[DPT], rg[DPT], rl[DPT], rv[NC];
  auto fetch = [&](int c0) {                    // global loads of the group that starts at token c0, into registers
    const int ct = min(CT, n - c0);
    if (tid < qk_items) {
      const int t = tid / R, rr = tid - t * R;
      const long row = tok0 + c0 + t;
      const int i0 = rr * DPT;
      if (t < ct && vec && i0 + DPT <= D) {
        if (!lower) ldn<T, DPT>(k + row * ldk + h * D + i0, rk);
        else ldn<float, DPT>(lower + h * D + i0, rl);
        ldn<T, DPT>(q + row * ldq + h * D + i0, rq);
        if (chan) {
          ldn<float, DPT>(z + row * ldz + h * D + i0, rg);
          float bb[DPT];
          ldn<float, DPT>(zb + h * D + i0, bb);
#pragma unroll
          for (int d = 0; d < DPT; ++d) rg[d] += bb[d];
        }
      } else {
#pragma unroll
        for (int d = 0; d < DPT; ++d) {
          const bool in = t < ct && i0 + d < D;
          rk[d] = (in && !lower) ? ldf(k + row * ldk + h * D + i0 + d) : 0.f;
          if (lower) rl[d] = in ? lower[h * D + i0 + d] : 1.f;                              // a = 1, k = 0: the state stays
          rq[d] = in ? ldf(q + row * ldq + h * D + i0 + d) : 0.f;
          if (chan) rg[d] = in ? z[row * ldz + h * D + i0 + d] + zb[h * D + i0 + d] : 1e30f;   // sigmoid(huge) = 1: no decay
        }
      }
    }
    if (tid < v_items) {
      const int t = tid / (VT / NC), cg = tid - t * (VT / NC);
      const long row = tok0 + c0 + t;
      const int col = j0 + cg * NC;
      if (t < ct && vec && col + NC <= V) {
        ldn<T, NC>(v + row * ldv + h * V + col, rv);
      } else {
#pragma unroll
        for (int c = 0; c < NC; ++c) rv[c] = (t < ct && col + c < V) ? ldf(v + row * ldv + h * V + col + c) : 0.f;
      }
    }
  };
  auto stash = [&](float* buf) {                // registers -> shared memory, with activations, scales and decays applied
    float* sk = buf; float* sq = sk + CT * Dp; float* sg = sq + CT * Dp; float* sv = sg + (chan ? CT * Dp : 0);
    if (tid < qk_items) {
      const int t = tid / R, rr = tid - t * R;
      float ko[DPT], qo[DPT], go[DPT];
#pragma unroll
      for (int d = 0; d < DPT; ++d) {
        float kv = rk[d], qv = rq[d];
        if (act & 1) qv = siluf_(qv);
        if (act & 2) kv = siluf_(kv);
        go[d] = chan ? expf(inv_tau * logsigmoidf_(rg[d])) : 1.f;
        if (lower) {
          go[d] = rl[d] + (1.f - rl[d]) * sigmoidf_(rg[d]);
          kv = 1.f - go[d];
        }
        ko[d] = kv * k_scale; qo[d] = qv * q_scale;
      }
#pragma unroll
      for (int d4 = 0; d4 < DPT / 4; ++d4) {
        reinterpret_cast<float4*>(sk + t * Dp + rr * PS)[d4] = make_float4(ko[4 * d4], ko[4 * d4 + 1], ko[4 * d4 + 2], ko[4 * d4 + 3]);
        reinterpret_cast<float4*>(sq + t * Dp + rr * PS)[d4] = make_float4(qo[4 * d4], qo[4 * d4 + 1], qo[4 * d4 + 2], qo[4 * d4 + 3]);
        if (chan) reinterpret_cast<float4*>(sg + t * Dp + rr * PS)[d4] = make_float4(go[4 * d4], go[4 * d4 + 1], go[4 * d4 + 2], go[4 * d4 + 3]);
      }
    }
    if (tid < v_items) {
      float vo[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) vo[c] = (act & 4) ? siluf_(rv[c]) : rv[c];
      reinterpret_cast<float4*>(sv)[2 * tid] = make_float4(vo[0], vo[1], vo[2], vo[3]);
      reinterpret_cast<float4*>(sv)[2 * tid + 1] = make_float4(vo[4], vo[5], vo[6], vo[7]);
    }
  };
  fetch(0);
  stash(sm);
  __syncthreads();
  int cur = 0;
  for (int c0 = 0; c0 < n; c0 += CT) {
    const int ct = min(CT, n - c0);
    const bool more = c0 + CT < n;
    if (more) fetch(c0 + CT);                   // in flight during the serial walk below
    asm volatile("" ::: "memory");              // (the loads may not sink below this point, towards their use after the walk)
    const float* buf = sm + cur * buf_floats;
    const float* sk = buf + r * PS; const float* sq = sk + CT * Dp; const float* sg = sq + CT * Dp;
    const float* sv = buf + CT * Dp * (chan ? 3 : 2) + (grp_ok ? grp * NC : 0);
    float* orow = out + (tok0 + c0) * (long)(H * V) + h * V;
    // every thread walks the tokens (lanes of idle column groups included: the shuffles below name the whole warp)
#pragma unroll 2
    for (int t = 0; t < ct; ++t, sk += Dp, sq += Dp, sg += Dp, sv += VT, orow += H * V) {
      const float4 va = reinterpret_cast<const float4*>(sv)[0], vb = reinterpret_cast<const float4*>(sv)[1];
      const float vt[NC] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
      float o[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) o[c] = 0.f;
#pragma unroll
      for (int d4 = 0; d4 < DPT / 4; ++d4) {
        const float4 kx = reinterpret_cast<const float4*>(sk)[d4], qx = reinterpret_cast<const float4*>(sq)[d4];
        float4 gx = make_float4(g0, g0, g0, g0);
        if (chan) gx = reinterpret_cast<const float4*>(sg)[d4];
        const float kk[4] = {kx.x, kx.y, kx.z, kx.w}, qq[4] = {qx.x, qx.y, qx.z, qx.w}, gg[4] = {gx.x, gx.y, gx.z, gx.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            s[4 * d4 + e][c] = s[4 * d4 + e][c] * gg[e] + kk[e] * vt[c];
            o[c] += s[4 * d4 + e][c] * qq[e];
          }
        }
      }
      if (R >= 8) {
        // transposing butterfly: after three rounds a lane holds, for one column, the sum over its 8 neighbouring lanes
        const bool b0 = r & 1, b1 = r & 2, b2 = r & 4;
        float a[4], bq[2];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = (b0 ? o[4 + i] : o[i]) + __shfl_xor_sync(0xffffffffu, b0 ? o[i] : o[4 + i], 1);
#pragma unroll
        for (int i = 0; i < 2; ++i) bq[i] = (b1 ? a[2 + i] : a[i]) + __shfl_xor_sync(0xffffffffu, b1 ? a[i] : a[2 + i], 2);
        float w = (b2 ? bq[1] : bq[0]) + __shfl_xor_sync(0xffffffffu, b2 ? bq[0] : bq[1], 4);
        for (int m = 8; m < R; m <<= 1) w += __shfl_xor_sync(0xffffffffu, w, m);
        const int col = jc + (b0 ? 4 : 0) + (b1 ? 2 : 0) + (b2 ? 1 : 0);
        if (r < 8 && grp_ok && col < V) orow[col] = w;
      } else {
        for (int m = R >> 1; m > 0; m >>= 1) {
#pragma unroll
          for (int c = 0; c < NC; ++c) o[c] += __shfl_xor_sync(0xffffffffu, o[c], m);
        }
        if (r == 0 && grp_ok) {
#pragma unroll
          for (int c = 0; c < NC; ++c) if (jc + c < V) orow[jc + c] = o[c];
        }
      }
    }
    if (more) stash(sm + (cur ^ 1) * buf_floats);
    __syncthreads();                            // the other buffer is complete, and nobody reads this one any more
    cur ^= 1;
  }
  if (grp_ok) {
#pragma unroll
    for (int d = 0; d < DPT; ++d) {
      const int i = r * DPT + d;
#pragma unroll
      for (int c = 0; c < NC; ++c) if (i < D && jc + c < V) Sg[(long)i * V + jc + c] = s[d][c];
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Gated RMS norm of a read-out o [rows, H*V] (fp32):  y = o / sqrt(mean(o^2) + eps) * w * act(gate) * out_scale, the
// mean taken over the V channels of every head (per_head = 1, w [V] shared by the heads or absent) or over the whole
// row (per_head = 0, w [H*V] or absent); act 0: silu, 1: sigmoid, 2: no gate (the gate pointer is not read).  One warp per
// (row, head), or one block per row.
// ------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void gated_norm_head_kernel(const float* __restrict__ o, const T* __restrict__ gate, long ldg, const T* __restrict__ w,
                                       float eps, int act, float out_scale, T* __restrict__ y, long ldy, long rows, int H, int V, int vec) {
  const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= rows * H) return;
  const long tok = wid / H; const int h = (int)(wid - tok * H);
  const float* orow = o + (tok * H + h) * (long)V;
  float ss = 0.f;
  if (vec) {                                     // four channels per lane and access (the second pass re-reads o from L1)
    for (int i = lane * 4; i < V; i += 128) { const float4 a = *reinterpret_cast<const float4*>(orow + i); ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w; }
    ss = warp_sum(ss);
    const float rv = out_scale / sqrtf(ss / (float)V + eps);
    for (int i = lane * 4; i < V; i += 128) {
      const float4 a = *reinterpret_cast<const float4*>(orow + i), g = act == 2 ? make_float4(0.f, 0.f, 0.f, 0.f) : ld4(gate + tok * ldg + h * V + i);
      const float4 wv = w ? ld4(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
      const float4 ga = act == 2 ? make_float4(1.f, 1.f, 1.f, 1.f)
                      : act == 0 ? make_float4(siluf_(g.x), siluf_(g.y), siluf_(g.z), siluf_(g.w))
                                 : make_float4(sigmoidf_(g.x), sigmoidf_(g.y), sigmoidf_(g.z), sigmoidf_(g.w));
      st4(y + tok * ldy + h * V + i, make_float4(a.x * rv * wv.x * ga.x, a.y * rv * wv.y * ga.y, a.z * rv * wv.z * ga.z, a.w * rv * wv.w * ga.w));
    }
    return;
  }
  for (int i = lane; i < V; i += 32) ss += orow[i] * orow[i];
  ss = warp_sum(ss);
  const float rr = out_scale / sqrtf(ss / (float)V + eps);
  for (int i = lane; i < V; i += 32) {
    const float g = act == 2 ? 0.f : ldf(gate + tok * ldg + h * V + i);
    const float ga = act == 2 ? 1.f : (act == 0 ? siluf_(g) : sigmoidf_(g));
    stf(y + tok * ldy + h * V + i, orow[i] * rr * (w ? ldf(w + i) : 1.f) * ga);
  }
}

template <typename T>
__global__ void gated_norm_row_kernel(const float* __restrict__ o, const T* __restrict__ gate, long ldg, const T* __restrict__ w,
                                      float eps, int act, float out_scale, T* __restrict__ y, long ldy, int n, int vec) {
  __shared__ float red[32];
  const long tok = blockIdx.x;
  const float* orow = o + tok * (long)n;
  float ss = 0.f;
  if (vec) {
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) { const float4 a = *reinterpret_cast<const float4*>(orow + i); ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w; }
    ss = block_sum(ss, red);
    const float rv = out_scale / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
      const float4 a = *reinterpret_cast<const float4*>(orow + i), g = act == 2 ? make_float4(0.f, 0.f, 0.f, 0.f) : ld4(gate + tok * ldg + i);
      const float4 wv = w ? ld4(w + i) : make_float4(1.f, 1.f, 1.f, 1.f);
      const float4 ga = act == 2 ? make_float4(1.f, 1.f, 1.f, 1.f)
                      : act == 0 ? make_float4(siluf_(g.x), siluf_(g.y), siluf_(g.z), siluf_(g.w))
                                 : make_float4(sigmoidf_(g.x), sigmoidf_(g.y), sigmoidf_(g.z), sigmoidf_(g.w));
      st4(y + tok * ldy + i, make_float4(a.x * rv * wv.x * ga.x, a.y * rv * wv.y * ga.y, a.z * rv * wv.z * ga.z, a.w * rv * wv.w * ga.w));
    }
    return;
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += orow[i] * orow[i];
  ss = block_sum(ss, red);
  const float rr = out_scale / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float g = act == 2 ? 0.f : ldf(gate + tok * ldg + i);
    const float ga = act == 2 ? 1.f : (act == 0 ? siluf_(g) : sigmoidf_(g));
    stf(y + tok * ldy + i, orow[i] * rr * (w ? ldf(w + i) : 1.f) * ga);
  }
}

}  // namespace

// ====================================================================================================================
// launchers (C ABI; return 0, a CUDA error code, or -1 for sizes a kernel is not built for)
// ====================================================================================================================
#define LAUNCH_END() do { const cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : (int)e_; } while (0)

extern "C" {

int lbl_embed_bigram(const void* table, const void* bigram, const int64_t* ids, int* last, const int* tok_seq, const int* seq_off,
                     const int* slots, const int* past, float scale, long mul_prev, long mul_cur, long buckets, float* x, long rows,
                     int n, int ns, int B, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  const int vec = (n % 4 == 0 && ((uintptr_t)table & 15) == 0 && ((uintptr_t)bigram & 15) == 0 && ((uintptr_t)x & 15) == 0) ? 1 : 0;
  const int threads = n >= 1024 ? 256 : 128;
  if (dtype) embed_bigram_kernel<bf16><<<(unsigned)rows, threads, 0, s>>>((const bf16*)table, (const bf16*)bigram, ids, last, tok_seq,
      seq_off, slots, past, scale, mul_prev, mul_cur, buckets, x, rows, n, ns, vec);
  else embed_bigram_kernel<float><<<(unsigned)rows, threads, 0, s>>>((const float*)table, (const float*)bigram, ids, last, tok_seq,
      seq_off, slots, past, scale, mul_prev, mul_cur, buckets, x, rows, n, ns, vec);
  token_last_kernel<<<(B + 127) / 128, 128, 0, s>>>(ids, last, seq_off, slots, B);
  LAUNCH_END();
}

int lbl_hc_step(float* x, long rows, int n, int ns, const void* y, long ldy, int ydtype, const int* pos, const float* cw, int top,
                const float* mix, const float* outw, const float* inw, const void* w, float eps, void* h, long ldh, int dtype,
                cudaStream_t s) {
  if (rows == 0) return 0;
  if (ns < 1 || ns > HC_MAXS) return -1;
  const size_t smem = h ? (size_t)n * sizeof(float) : 0;
  if (smem > 160 * 1024) return -1;
  int vec = (n % 4 == 0 && ((uintptr_t)x & 15) == 0) ? 1 : 0;
  if (y && (((uintptr_t)y & 15) != 0 || ldy % 4 != 0)) vec = 0;
  if (h && (((uintptr_t)h & 15) != 0 || ldh % 4 != 0 || ((uintptr_t)w & 15) != 0)) vec = 0;
  const int quads = n / 4;
  if (vec && ns <= 4 && quads <= 2048) {          // every quadruple of the row in registers: at most two per thread
    const int items = quads <= 128 ? 1 : 2;
    const int vthreads = (((quads + items - 1) / items + 31) / 32) * 32;
    const int nsb = ns <= 1 ? 1 : (ns <= 2 ? 2 : 4);
#define HCV3(TT, TY, NSB, IT) hc_step_vec_kernel<TT, TY, NSB, IT><<<(unsigned)rows, vthreads, 0, s>>>(x, rows, n, ns, (const TY*)y, ldy, pos, cw, \
        top, mix, outw, inw, (const TT*)w, eps, (TT*)h, ldh)
#define HCV2(TT, TY, NSB) { if (items == 1) HCV3(TT, TY, NSB, 1); else HCV3(TT, TY, NSB, 2); }
#define HCV(TT, TY) { if (nsb == 1) HCV2(TT, TY, 1) else if (nsb == 2) HCV2(TT, TY, 2) else HCV2(TT, TY, 4) }
    if (dtype) { if (ydtype) HCV(bf16, bf16) else HCV(bf16, float) }
    else { if (ydtype) return -1; HCV(float, float) }
#undef HCV
#undef HCV2
#undef HCV3
    LAUNCH_END();
  }
  const int threads = n >= 2048 ? 256 : 128;
#define HC(TT, TY) { \
    if (smem > 48 * 1024) cudaFuncSetAttribute(hc_step_kernel<TT, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    hc_step_kernel<TT, TY><<<(unsigned)rows, threads, smem, s>>>(x, rows, n, ns, (const TY*)y, ldy, pos, cw, top, mix, outw, inw, \
                                                                 (const TT*)w, eps, (TT*)h, ldh); }
  if (dtype) { if (ydtype) HC(bf16, bf16) else HC(bf16, float) }
  else { if (ydtype) return -1; HC(float, float) }
#undef HC
  LAUNCH_END();
}

int lbl_decay_scan(const void* q, long ldq, const void* k, long ldk, const void* v, long ldv, const float* decay, const float* z,
                   long ldz, const float* zb, const float* lower, float inv_tau, float q_scale, float k_scale, int act, float* S,
                   const int* seq_off, const int* slots, const int* past, float* out, int B, int H, int D, int V, int dtype,
                   cudaStream_t s) {
  if (B == 0) return 0;
  if (D > 256 || (!decay && !z) || (z && !zb) || (lower && !z)) return -1;
  int dpt = D <= 64 ? 4 : 8;                    // rows per lane: 16 lanes per column group at D = 64 and at D = 128
  // few (sequence, head) pairs: the smaller tile doubles the threads per pair, which hides more of the serial walk's latency
  if (dpt == 8 && D <= 128 && (long)B * H * ((V + 127) / 128) < 100) dpt = 4;
  int R = 1;
  while (R * dpt < D) R <<= 1;                  // lanes per column group: a power of two <= 32
  const int groups_max = 256 / R;               // column groups of 8 columns in a block of 256 threads
  int groups = (V + SCAN_NC - 1) / SCAN_NC;
  if (groups > groups_max) groups = groups_max;
  // columns are independent: smaller blocks when one block per (sequence, head) would leave most SMs idle
  while (groups > 2 && groups % 2 == 0 && (long)B * H * ((V + groups * SCAN_NC - 1) / (groups * SCAN_NC)) < 100) groups /= 2;
  const int VT = groups * SCAN_NC;
  const int threads = ((groups * R + 31) / 32) * 32;
  int CT = SCAN_CT;                             // tokens per staged group: one (token, lane chunk) and one (token, column group) per thread
  while (CT > 1 && (CT * R > threads || CT * groups > threads)) CT >>= 1;
  const int Dp = R * (dpt == 8 ? 12 : 4);
  const size_t smem = 2 * sizeof(float) * (size_t)CT * ((size_t)Dp * (z ? 3 : 2) + VT);
  const dim3 grid((unsigned)(B * H), (unsigned)((V + VT - 1) / VT));
  const int esz = dtype ? 2 : 4;
  const int vec = (D % 8 == 0 && V % 8 == 0 && (ldq * esz) % 16 == 0 && (ldk * esz) % 16 == 0 && (ldv * esz) % 16 == 0 &&
                   ((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0 && ((uintptr_t)v & 15) == 0 &&
                   (!z || (ldz % 4 == 0 && ((uintptr_t)z & 15) == 0 && ((uintptr_t)zb & 15) == 0)) && ((uintptr_t)lower & 15) == 0) ? 1 : 0;
#define DS(TT, P) { \
    if (smem > 48 * 1024) cudaFuncSetAttribute(decay_scan_kernel<TT, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    decay_scan_kernel<TT, P><<<grid, threads, smem, s>>>((const TT*)q, ldq, (const TT*)k, ldk, (const TT*)v, ldv, decay, z, ldz, zb, lower, \
        inv_tau, q_scale, k_scale, act, S, seq_off, slots, past, out, H, D, V, R, VT, CT, vec); }
  if (dtype == 0) { if (dpt == 4) DS(float, 4) else DS(float, 8) }
  else { if (dpt == 4) DS(bf16, 4) else DS(bf16, 8) }
#undef DS
  LAUNCH_END();
}

int lbl_gated_norm(const float* o, const void* gate, long ldg, const void* w, float eps, int act, float out_scale, void* y, long ldy,
                   long rows, int H, int V, int per_head, int dtype, cudaStream_t s) {
  if (rows == 0) return 0;
  if (act == 2) { gate = nullptr; ldg = 0; }
  const int vec = (V % 4 == 0 && ldg % 4 == 0 && ldy % 4 == 0 && ((uintptr_t)o & 15) == 0 && ((uintptr_t)gate & 15) == 0 &&
                   ((uintptr_t)y & 15) == 0 && ((uintptr_t)w & 15) == 0) ? 1 : 0;
  if (per_head) {
    const unsigned grid = (unsigned)((rows * H * 32 + 255) / 256);
    if (dtype) gated_norm_head_kernel<bf16><<<grid, 256, 0, s>>>(o, (const bf16*)gate, ldg, (const bf16*)w, eps, act, out_scale, (bf16*)y, ldy, rows, H, V, vec);
    else gated_norm_head_kernel<float><<<grid, 256, 0, s>>>(o, (const float*)gate, ldg, (const float*)w, eps, act, out_scale, (float*)y, ldy, rows, H, V, vec);
  } else {
    const int n = H * V, threads = n >= 1024 ? 256 : 128;
    if (dtype) gated_norm_row_kernel<bf16><<<(unsigned)rows, threads, 0, s>>>(o, (const bf16*)gate, ldg, (const bf16*)w, eps, act, out_scale, (bf16*)y, ldy, n, vec);
    else gated_norm_row_kernel<float><<<(unsigned)rows, threads, 0, s>>>(o, (const float*)gate, ldg, (const float*)w, eps, act, out_scale, (float*)y, ldy, n, vec);
  }
  LAUNCH_END();
}

}  // extern "C"
