// torch.ops.libai_b200_lin.* : argument-checking wrappers around the launchers of lin_mixers.cu (token + bigram embedding,
// hyper-connection streams, decayed linear-attention recurrences, gated read-out norms).  A library of its own so that a model
// that only needs these kernels builds nothing else.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

extern "C" {
int lbl_embed_bigram(const void* table, const void* bigram, const int64_t* ids, int* last, const int* tok_seq, const int* seq_off,
                     const int* slots, const int* past, float scale, long mul_prev, long mul_cur, long buckets, float* x, long rows,
                     int n, int ns, int B, int dtype, cudaStream_t s);
int lbl_hc_step(float* x, long rows, int n, int ns, const void* y, long ldy, int ydtype, const int* pos, const float* cw, int top,
                const float* mix, const float* outw, const float* inw, const void* w, float eps, void* h, long ldh, int dtype,
                cudaStream_t s);
int lbl_decay_scan(const void* q, long ldq, const void* k, long ldk, const void* v, long ldv, const float* decay, const float* z,
                   long ldz, const float* zb, const float* lower, float inv_tau, float q_scale, float k_scale, int act, float* S,
                   const int* seq_off, const int* slots, const int* past, float* out, int B, int H, int D, int V, int dtype,
                   cudaStream_t s);
int lbl_gated_norm(const float* o, const void* gate, long ldg, const void* w, float eps, int act, float out_scale, void* y, long ldy,
                   long rows, int H, int V, int per_head, int dtype, cudaStream_t s);
}

namespace {
using at::Tensor;
using OptT = c10::optional<Tensor>;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void check(int err, const char* what) {
  TORCH_CHECK(err == 0, what, err < 0 ? ": unsupported sizes" : ": CUDA error ", err < 0 ? "" : cudaGetErrorString((cudaError_t)err));
}
int code(const Tensor& t) {
  TORCH_CHECK(t.scalar_type() == at::kFloat || t.scalar_type() == at::kBFloat16, "float32 or bfloat16 expected");
  return t.scalar_type() == at::kFloat ? 0 : 1;
}
void rows2d(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 2 && (t.size(1) == 1 || t.stride(1) == 1), name, ": 2-D CUDA tensor with unit column stride expected");
}
const int* meta(const Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), "int32 CUDA metadata expected");
  return t.data_ptr<int>();
}
bool has(const OptT& t) { return t.has_value() && t->defined(); }
const float* f32(const Tensor& t, int64_t n, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous() && t.numel() == n, name, ": contiguous fp32 tensor of the stated size expected");
  return t.data_ptr<float>();
}

// x [streams, rows, n] fp32 receives table[ids] * scale + bigram[row] in every stream; `last` int32 [slots] is the previous
// token of every sequence (read for a step's first row when past > 0, then set to the step's last token)
void embed_bigram(const Tensor& table, const Tensor& bigram, const Tensor& ids, Tensor last, const Tensor& tok_seq, const Tensor& seq_off,
                  const Tensor& slots, const Tensor& past, double scale, int64_t mul_prev, int64_t mul_cur, int64_t buckets, Tensor x) {
  TORCH_CHECK(table.is_cuda() && table.dim() == 2 && table.is_contiguous() && bigram.dim() == 2 && bigram.is_contiguous() &&
              bigram.size(1) == table.size(1) && bigram.size(0) == buckets + 1 && code(table) == code(bigram), "embed_bigram: tables");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "embed_bigram: int64 ids expected");
  TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.is_contiguous() && x.scalar_type() == at::kFloat && x.size(1) == ids.numel() &&
              x.size(2) == table.size(1), "embed_bigram: x fp32 [streams, rows, width]");
  TORCH_CHECK(last.is_cuda() && last.scalar_type() == at::kInt && last.is_contiguous(), "embed_bigram: last int32 [slots]");
  c10::cuda::CUDAGuard guard(table.device());
  check(lbl_embed_bigram(table.data_ptr(), bigram.data_ptr(), ids.data_ptr<int64_t>(), last.data_ptr<int>(), meta(tok_seq), meta(seq_off),
                         meta(slots), meta(past), (float)scale, (long)mul_prev, (long)mul_cur, (long)buckets, x.data_ptr<float>(),
                         ids.numel(), (int)table.size(1), (int)x.size(0), (int)slots.numel(), code(table), cur_stream()), "embed_bigram");
}

void hc_step(Tensor x, const OptT& y, const OptT& pos, const OptT& cw, const OptT& mix, const OptT& outw, const OptT& inw, const OptT& w,
             double eps, const OptT& h) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.is_contiguous() && x.scalar_type() == at::kFloat, "hc_step: x fp32 [streams, rows, width]");
  const int64_t ns = x.size(0), rows = x.size(1), n = x.size(2);
  const void* yp = nullptr; long ldy = 0; int ydtype = 0, top = 0;
  const int* pp = nullptr; const float* cp = nullptr; const float* mp = nullptr; const float* op = nullptr;
  if (has(y)) {
    rows2d(*y, "hc_step y");
    TORCH_CHECK(y->size(1) == n && has(mix) && has(outw), "hc_step: y [rows, width] with mix and out");
    yp = y->data_ptr(); ldy = y->stride(0); ydtype = code(*y);
    mp = f32(*mix, ns * ns, "hc_step mix"); op = f32(*outw, ns, "hc_step out");
    if (has(pos)) {
      TORCH_CHECK(has(cw) && pos->numel() == cw->numel() && pos->numel() % std::max<int64_t>(rows, 1) == 0, "hc_step: pos / cw [rows, top]");
      pp = meta(*pos); top = (int)(pos->numel() / std::max<int64_t>(rows, 1)); cp = f32(*cw, pos->numel(), "hc_step cw");
    } else {
      TORCH_CHECK(y->size(0) == rows, "hc_step: y rows");
    }
  }
  void* hp = nullptr; long ldh = 0; const float* ip = nullptr; const void* wp = nullptr; int dtype = 0;
  if (has(h)) {
    rows2d(*h, "hc_step h");
    TORCH_CHECK(h->size(0) == rows && h->size(1) == n && has(inw) && has(w) && w->is_contiguous() && w->numel() == n && code(*w) == code(*h),
                "hc_step: h [rows, width] with in and the norm weight");
    hp = h->data_ptr(); ldh = h->stride(0); ip = f32(*inw, ns, "hc_step in"); wp = w->data_ptr(); dtype = code(*h);
  } else if (has(y)) {
    dtype = ydtype;
  }
  c10::cuda::CUDAGuard guard(x.device());
  check(lbl_hc_step(x.data_ptr<float>(), rows, (int)n, (int)ns, yp, ldy, ydtype, pp, cp, top, mp, op, ip, wp, (float)eps, hp, ldh, dtype,
                    cur_stream()), "hc_step");
}

void decay_scan(const Tensor& q, const Tensor& k, const Tensor& v, const OptT& decay, const OptT& z, const OptT& zb, double inv_tau,
                double q_scale, double k_scale, int64_t act, Tensor S, const Tensor& seq_off, const Tensor& slots, const Tensor& past, Tensor out,
                const OptT& lower) {
  rows2d(q, "decay_scan q"); rows2d(k, "decay_scan k"); rows2d(v, "decay_scan v");
  TORCH_CHECK(S.is_cuda() && S.dim() == 4 && S.is_contiguous() && S.scalar_type() == at::kFloat, "decay_scan: S must be fp32 [slots, H, D, V]");
  const int H = (int)S.size(1), D = (int)S.size(2), V = (int)S.size(3);
  TORCH_CHECK(q.size(1) == (long)H * D && k.size(1) == (long)H * D && v.size(1) == (long)H * V && k.size(0) == q.size(0) && v.size(0) == q.size(0) &&
              code(q) == code(k) && code(q) == code(v), "decay_scan: q, k [tokens, H*D], v [tokens, H*V] of one dtype");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.is_contiguous() && out.dim() == 2 && out.size(1) == (long)H * V &&
              out.size(0) == q.size(0), "decay_scan: out must be fp32 [tokens, H*V]");
  const float* dp = nullptr; const float* zp = nullptr; const float* bp = nullptr; const float* lp = nullptr; long ldz = 0;
  if (has(lower)) { TORCH_CHECK(has(z), "decay_scan: a lower bound needs decay logits"); lp = f32(*lower, (int64_t)H * D, "decay_scan lower"); }
  if (has(z)) {
    rows2d(*z, "decay_scan z");
    TORCH_CHECK(z->scalar_type() == at::kFloat && z->size(0) == q.size(0) && z->size(1) == (long)H * D && has(zb), "decay_scan: z fp32 [tokens, H*D] with its bias");
    zp = z->data_ptr<float>(); ldz = z->stride(0); bp = f32(*zb, (int64_t)H * D, "decay_scan zb");
  } else {
    TORCH_CHECK(has(decay), "decay_scan: a decay per head or decay logits per key channel");
    dp = f32(*decay, H, "decay_scan decay");
  }
  c10::cuda::CUDAGuard guard(q.device());
  check(lbl_decay_scan(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), dp, zp, ldz, bp, lp, (float)inv_tau,
                       (float)q_scale, (float)k_scale, (int)act, S.data_ptr<float>(), meta(seq_off), meta(slots), meta(past),
                       out.data_ptr<float>(), (int)slots.numel(), H, D, V, code(q), cur_stream()), "decay_scan");
}

void gated_norm(const Tensor& o, const OptT& gate_opt, const OptT& w, double eps, int64_t act, double out_scale, Tensor y, int64_t H, int64_t V,
                bool per_head) {
  TORCH_CHECK(has(gate_opt) || act == 2, "gated_norm: a gate, or act 2 (none)");
  const Tensor& gate = has(gate_opt) ? *gate_opt : y;      // act 2 reads no gate
  rows2d(gate, "gated_norm gate"); rows2d(y, "gated_norm y");
  TORCH_CHECK(o.is_cuda() && o.scalar_type() == at::kFloat && o.is_contiguous() && o.numel() == y.size(0) * H * V, "gated_norm: o fp32 [rows, H*V]");
  TORCH_CHECK(gate.size(1) == H * V && gate.size(0) == y.size(0) && y.size(1) == H * V && code(gate) == code(y), "gated_norm: shapes");
  const void* wp = nullptr;
  if (has(w)) {
    TORCH_CHECK(w->is_cuda() && w->is_contiguous() && w->numel() == (per_head ? V : H * V) && code(*w) == code(y), "gated_norm: weight");
    wp = w->data_ptr();
  }
  c10::cuda::CUDAGuard guard(o.device());
  check(lbl_gated_norm(o.data_ptr<float>(), gate.data_ptr(), gate.stride(0), wp, (float)eps, (int)act, (float)out_scale, y.data_ptr(),
                       y.stride(0), y.size(0), (int)H, (int)V, per_head ? 1 : 0, code(y), cur_stream()), "gated_norm");
}
}  // namespace

TORCH_LIBRARY(libai_b200_lin, m) {
  m.def("embed_bigram(Tensor table, Tensor bigram, Tensor ids, Tensor(a!) last, Tensor tok_seq, Tensor seq_off, Tensor slots, Tensor past, float scale, int mul_prev, int mul_cur, int buckets, Tensor(b!) x) -> ()", &embed_bigram);
  m.def("hc_step(Tensor(a!) x, Tensor? y, Tensor? pos, Tensor? cw, Tensor? mix, Tensor? outw, Tensor? inw, Tensor? w, float eps, Tensor(b!)? h) -> ()", &hc_step);
  m.def("decay_scan(Tensor q, Tensor k, Tensor v, Tensor? decay, Tensor? z, Tensor? zb, float inv_tau, float q_scale, float k_scale, int act, Tensor(a!) S, Tensor seq_off, Tensor slots, Tensor past, Tensor(b!) out, Tensor? lower=None) -> ()", &decay_scan);
  m.def("gated_norm(Tensor o, Tensor? gate, Tensor? w, float eps, int act, float out_scale, Tensor(a!) y, int H, int V, bool per_head) -> ()", &gated_norm);
}
