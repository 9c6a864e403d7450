// torch.ops.libai_b200_kv.* : argument-checking wrappers around the launchers of kv_mixers.cu (Dynamic-Tanh norms, query/key
// preparation, ring key/value caches, masked grouped-query attention, mixture-of-experts feed-forward) and of paged_mixers.cu
// (post-norm residual, convolved query/key/value preparation into a paged cache, attention over the pages with mixed heads
// and a learned sink).  A library of its own so that a model that only needs these kernels builds nothing else.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

extern "C" {
int lbk_embed_scale(const void* table, const int64_t* ids, float scale, float* x, long rows, int n, int dtype, cudaStream_t s);
int lbk_dyt_residual(float* x, const void* y, long ldy, int ydtype, const int* pos, const float* cw, int top, const void* pw,
                     const void* pb, const void* palpha, const void* nw, const void* nb, const void* nalpha, void* h, long ldh,
                     long rows, int n, int dtype, cudaStream_t s);
int lbk_act_rows(const void* in, long ldi, void* out, long ldo, long rows, int n, int act, int gated, float limit, int dtype,
                 cudaStream_t s);
int lbk_softcap(float* l, float cap, long total, cudaStream_t s);
int lbk_qk_prepare(void* q, long ldq, void* k, long ldk, const void* qw, const void* kw, const float* freq, float mscale, int rot,
                   int H, int G, int D, float eps, int full_norm, int unit_norm, const int* tok_seq, const int* seq_off,
                   const int* past, long tokens, int dtype, cudaStream_t s);
int lbk_kv_write(void* ring, void* first, const void* knew, const void* vnew, long ldn, const int* tok_seq, const int* seq_off,
                 const int* slots, const int* past, long tokens, int KC, int VC, int L, int nfirst, int dtype, cudaStream_t s);
int lbk_kv_gather(const void* ring, const void* first, const void* knew, const void* vnew, long ldn, const int* ext_seq,
                  const int* ext_off, const int* nsink, const int* cstart, const int* seq_off, const int* slots, const int* past,
                  void* ext, long rows, int KC, int VC, int L, int nfirst, int dtype, cudaStream_t s);
int lbk_masked_attention(const void* q, long ldq, const void* kbase, const void* vbase, long ldkv, const void* ring, const void* first,
                         int L, int nfirst, const int* ext_off, const int* nsink, const int* cstart, const int* slots,
                         const void* gate, long ldg, const int* tok_seq, const int* seq_off, const int* past, void* y, long ldy,
                         long tokens, int H, int G, int D, int V, int window, int chunk, int keep, float scale, float softcap,
                         int sink, int gate_wide, float out_scale, int dtype, cudaStream_t s);
int lbk_masked_attention_mma(const void* q, long ldq, const void* kbase, const void* vbase, long ldkv, const int* ext_off,
                             const int* nsink, const int* cstart, const void* gate, long ldg, const int* qt_seq, const int* qt_start,
                             int n_qtiles, const int* seq_off, const int* past, void* y, long ldy, int H, int G, int D, int V,
                             int window, int chunk, int keep, float scale, float softcap, int sink, int gate_wide, float out_scale,
                             cudaStream_t s);
int lbk_ring_decode(const void* q, long ldq, const void* ring, const void* first, int L, int nfirst, const int* slots, const int* past,
                    const void* gate, long ldg, void* y, long ldy, float* part, int B, int H, int G, int D, int V, int window,
                    int chunk, int keep, float scale, int splits, float softcap, int sink, int gate_wide, float out_scale, int dtype,
                    cudaStream_t s);
int lbk_moe_topk(const float* z, long ldz, const float* bias, int mode, int E, int top, float rscale, int* idx, float* wts, int* counts,
                 long tokens, cudaStream_t s);
int lbk_moe_pairs(const void* h, long ldh, const void* wgu, const void* wd, const int* idx, const float* wts, void* a, float* out,
                  long tokens, int ff, int n, int top, int act, float limit, int win, int dtype, cudaStream_t s);
int lbk_moe_sort(const void* h, long ldh, const int* idx, const int* counts, int* offsets, int* cursor, int* pos, void* xs, long tokens,
                 int E, int n, int top, int align, int* tile_group, int tiles, const float* wts, int dtype, cudaStream_t s);
int lbp_postnorm_residual(const float* xin, float* xout, const void* y1, long ldy1, int y1dtype, const float* y2, long ldy2,
                          const int* pos, const float* cw, int top, float alpha, const void* w, float eps, void* h, long ldh,
                          long rows, int n, int dtype, cudaStream_t s);
int lbp_conv_qkv_prepare(const void* qin, const void* kin, const void* vin, long ld, const void* wq, const void* wk, const void* wv,
                         int taps, void* tail, const void* qn, const void* kn, const float* freq, int half, float eps, void* qout,
                         long ldqo, void* pool, const int* table, int max_pages, int page_size, const int* tok_seq,
                         const int* seq_off, const int* slots, const int* past, long tokens, int B, int H, int G, int D, int V,
                         int dtype, cudaStream_t s);
int lbp_talk_attention_tiles(int qt_max, int H, int G, int D, int V, int* kt_out);
int lbp_talk_attention_mma(const void* q, long ldq, const void* pool, const int* table, int max_pages, int page_size, const float* talk,
                           const float* sink, const int* qt_seq, const int* qt_start, int ntiles, const int* seq_off, const int* slots,
                           const int* past, void* y, long ldy, int H, int G, int D, int V, float scale, float out_scale, cudaStream_t s);
int lbp_talk_attention(const void* q, long ldq, const void* pool, const int* table, int max_pages, int page_size, const float* talk,
                       const float* sink, const int* qt_seq, const int* qt_start, int ntiles, int QT, int KT, const int* seq_off,
                       const int* slots, const int* past, void* y, long ldy, float* part, int nparts, long rows, int H, int G, int D,
                       int V, float scale, float out_scale, int dtype, cudaStream_t s);
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
const int* meta_opt(const OptT& t) { return (t.has_value() && t->defined()) ? meta(*t) : nullptr; }
const void* ptr_opt(const OptT& t) { return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr; }
bool has(const OptT& t) { return t.has_value() && t->defined(); }
void vec(const Tensor& t, int64_t n, int dtype, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.numel() == n && code(t) == dtype, name, ": contiguous vector of the model's dtype expected");
}

void embed_scale(const Tensor& table, const Tensor& ids, double scale, Tensor x) {
  TORCH_CHECK(table.is_cuda() && table.dim() == 2 && table.is_contiguous(), "embed_scale: contiguous table");
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "embed_scale: int64 ids expected");
  TORCH_CHECK(x.scalar_type() == at::kFloat && x.is_contiguous() && x.dim() == 2 && x.size(0) == ids.numel() && x.size(1) == table.size(1),
              "embed_scale: x fp32 [rows, width]");
  c10::cuda::CUDAGuard guard(x.device());
  check(lbk_embed_scale(table.data_ptr(), ids.data_ptr<int64_t>(), (float)scale, x.data_ptr<float>(), ids.numel(), (int)table.size(1),
                        code(table), cur_stream()), "embed_scale");
}

// x += dyt(y; pw, pb, palpha) (y optional; with `pos`/`cw` y is gathered: sum_k cw[r,k] * y[pos[r,k]]), h = dyt(x; nw, nb, nalpha) (optional)
void dyt_residual(Tensor x, const OptT& y, const OptT& pos, const OptT& cw, const OptT& pw, const OptT& pb, const OptT& palpha,
                  const OptT& nw, const OptT& nb, const OptT& nalpha, const OptT& h) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous() && x.dim() == 2, "dyt_residual: x fp32 [rows, width]");
  const int64_t rows = x.size(0), n = x.size(1);
  int dtype = -1, ydtype = 0, top = 0;
  long ldy = 0, ldh = 0;
  if (has(h)) {
    rows2d(*h, "dyt_residual h");
    dtype = code(*h); ldh = h->stride(0);
    TORCH_CHECK(h->size(0) == rows && h->size(1) == n && has(nw) && has(nb) && has(nalpha), "dyt_residual: h and its norm");
    vec(*nw, n, dtype, "dyt_residual nw"); vec(*nb, n, dtype, "dyt_residual nb"); vec(*nalpha, 1, dtype, "dyt_residual nalpha");
  }
  if (has(y)) {
    rows2d(*y, "dyt_residual y");
    TORCH_CHECK(has(pw) && has(pb) && has(palpha) && y->size(1) == n, "dyt_residual: y and its norm");
    if (dtype < 0) dtype = code(*pw);
    vec(*pw, n, dtype, "dyt_residual pw"); vec(*pb, n, dtype, "dyt_residual pb"); vec(*palpha, 1, dtype, "dyt_residual palpha");
    ydtype = code(*y); ldy = y->stride(0);
    if (has(pos)) {
      TORCH_CHECK(has(cw) && cw->is_cuda() && cw->scalar_type() == at::kFloat && cw->is_contiguous() && cw->numel() == pos->numel() &&
                  pos->numel() % rows == 0, "dyt_residual: pos / weights [rows, top]");
      top = (int)(pos->numel() / rows);
    } else {
      TORCH_CHECK(y->size(0) == rows, "dyt_residual: y rows");
    }
  }
  TORCH_CHECK(dtype >= 0, "dyt_residual: nothing to do");
  c10::cuda::CUDAGuard guard(x.device());
  check(lbk_dyt_residual(x.data_ptr<float>(), ptr_opt(y), ldy, ydtype, has(y) ? meta_opt(pos) : nullptr,
                         has(y) && has(pos) ? cw->data_ptr<float>() : nullptr, top, ptr_opt(pw), ptr_opt(pb), ptr_opt(palpha), ptr_opt(nw),
                         ptr_opt(nb), ptr_opt(nalpha), has(h) ? h->data_ptr() : nullptr, ldh, rows, (int)n, dtype, cur_stream()),
        "dyt_residual");
}

void act_rows(const Tensor& in, Tensor out, int64_t act, bool gated, double limit) {
  rows2d(in, "act_rows in"); rows2d(out, "act_rows out");
  TORCH_CHECK(in.size(0) == out.size(0) && in.size(1) == (gated ? 2 : 1) * out.size(1) && code(in) == code(out), "act_rows: shapes");
  c10::cuda::CUDAGuard guard(in.device());
  check(lbk_act_rows(in.data_ptr(), in.stride(0), out.data_ptr(), out.stride(0), out.size(0), (int)out.size(1), (int)act, gated ? 1 : 0,
                     (float)limit, code(in), cur_stream()), "act_rows");
}

void softcap(Tensor l, double cap) {
  TORCH_CHECK(l.is_cuda() && l.scalar_type() == at::kFloat && l.is_contiguous(), "softcap: contiguous fp32 expected");
  c10::cuda::CUDAGuard guard(l.device());
  check(lbk_softcap(l.data_ptr<float>(), (float)cap, l.numel(), cur_stream()), "softcap");
}

void qk_prepare(Tensor q, const OptT& k, const OptT& qw, const OptT& kw, const Tensor& freq, double mscale, int64_t H, int64_t G,
                int64_t D, double eps, bool full_norm, bool unit_norm, const Tensor& tok_seq, const Tensor& seq_off, const Tensor& past) {
  rows2d(q, "qk_prepare q");
  const int dtype = code(q);
  TORCH_CHECK(q.size(1) == H * D, "qk_prepare: q [tokens, H*D]");
  TORCH_CHECK(freq.is_cuda() && freq.scalar_type() == at::kFloat && freq.is_contiguous(), "qk_prepare: fp32 frequencies");
  if (has(k)) { rows2d(*k, "qk_prepare k"); TORCH_CHECK(k->size(1) == G * D && k->size(0) == q.size(0) && code(*k) == dtype, "qk_prepare: k [tokens, G*D]"); }
  if (full_norm) {
    TORCH_CHECK(has(qw), "qk_prepare: the whole-projection norm needs its weight");
    vec(*qw, H * D, dtype, "qk_prepare qw");
    if (has(k)) { TORCH_CHECK(has(kw), "qk_prepare: key norm weight"); vec(*kw, G * D, dtype, "qk_prepare kw"); }
  }
  c10::cuda::CUDAGuard guard(q.device());
  check(lbk_qk_prepare(q.data_ptr(), q.stride(0), has(k) ? k->data_ptr() : nullptr, has(k) ? k->stride(0) : 0, ptr_opt(qw), ptr_opt(kw),
                       freq.data_ptr<float>(), (float)mscale, (int)(2 * freq.numel()), (int)H, (int)G, (int)D, (float)eps, full_norm ? 1 : 0,
                       unit_norm ? 1 : 0, meta(tok_seq), meta(seq_off), meta(past), q.size(0), dtype, cur_stream()), "qk_prepare");
}

void ring_shapes(const Tensor& ring, const Tensor& first, int64_t C) {
  TORCH_CHECK(ring.is_cuda() && ring.dim() == 3 && ring.is_contiguous() && ring.size(2) == C, "ring [slots, L, C] expected");
  TORCH_CHECK(first.is_cuda() && first.dim() == 3 && first.is_contiguous() && first.size(2) == C && first.size(0) == ring.size(0) &&
              code(first) == code(ring), "first [slots, nfirst, C] expected");
}

void kv_write(Tensor ring, Tensor first, const Tensor& knew, const Tensor& vnew, const Tensor& tok_seq, const Tensor& seq_off,
              const Tensor& slots, const Tensor& past) {
  rows2d(knew, "kv_write k"); rows2d(vnew, "kv_write v");
  ring_shapes(ring, first, knew.size(1) + vnew.size(1));
  TORCH_CHECK(knew.stride(0) == vnew.stride(0) && knew.size(0) == vnew.size(0) && code(knew) == code(ring) && code(vnew) == code(ring),
              "kv_write: keys and values are column slices of one matrix");
  c10::cuda::CUDAGuard guard(ring.device());
  check(lbk_kv_write(ring.data_ptr(), first.data_ptr(), knew.data_ptr(), vnew.data_ptr(), knew.stride(0), meta(tok_seq), meta(seq_off),
                     meta(slots), meta(past), knew.size(0), (int)knew.size(1), (int)vnew.size(1), (int)ring.size(1), (int)first.size(1),
                     code(ring), cur_stream()), "kv_write");
}

void kv_gather(const Tensor& ring, const Tensor& first, const Tensor& knew, const Tensor& vnew, const Tensor& ext_seq,
               const Tensor& ext_off, const Tensor& nsink, const Tensor& cstart, const Tensor& seq_off, const Tensor& slots,
               const Tensor& past, Tensor ext) {
  rows2d(knew, "kv_gather k"); rows2d(vnew, "kv_gather v");
  ring_shapes(ring, first, knew.size(1) + vnew.size(1));
  TORCH_CHECK(ext.is_cuda() && ext.dim() == 2 && ext.is_contiguous() && ext.size(1) == ring.size(2) && code(ext) == code(ring) &&
              ext.size(0) == ext_seq.numel(), "kv_gather: ext [rows, C]");
  TORCH_CHECK(knew.stride(0) == vnew.stride(0) && code(knew) == code(ring) && code(vnew) == code(ring), "kv_gather: new rows");
  c10::cuda::CUDAGuard guard(ring.device());
  check(lbk_kv_gather(ring.data_ptr(), first.data_ptr(), knew.data_ptr(), vnew.data_ptr(), knew.stride(0), meta(ext_seq), meta(ext_off),
                      meta(nsink), meta(cstart), meta(seq_off), meta(slots), meta(past), ext.data_ptr(), ext.size(0), (int)knew.size(1),
                      (int)vnew.size(1), (int)ring.size(1), (int)first.size(1), code(ring), cur_stream()), "kv_gather");
}

// prompt steps: keys / values are column slices (kmat, vmat) of the ext matrix
void masked_attention(const Tensor& q, const Tensor& kmat, const Tensor& vmat, const Tensor& ext_off, const Tensor& nsink,
                      const Tensor& cstart, const OptT& gate, const Tensor& tok_seq, const Tensor& seq_off, const Tensor& past,
                      const OptT& qt_seq, const OptT& qt_start, Tensor y, int64_t H, int64_t G, int64_t D, int64_t V, int64_t window,
                      int64_t chunk, int64_t keep, double scale, double softcap, bool sink, bool gate_wide, double out_scale) {
  rows2d(q, "masked_attention q"); rows2d(kmat, "masked_attention k"); rows2d(vmat, "masked_attention v"); rows2d(y, "masked_attention y");
  const int dtype = code(q);
  TORCH_CHECK(q.size(1) == H * D && kmat.size(1) == G * D && vmat.size(1) == G * V && y.size(1) == H * V && y.size(0) == q.size(0) &&
              kmat.stride(0) == vmat.stride(0) && code(kmat) == dtype && code(vmat) == dtype && code(y) == dtype, "masked_attention: shapes");
  long ldg = 0;
  if (has(gate)) { rows2d(*gate, "masked_attention gate"); TORCH_CHECK(gate->size(1) == (gate_wide ? H * V : H) && code(*gate) == dtype, "masked_attention: gate [tokens, H] (or [tokens, H V])"); ldg = gate->stride(0); }
  c10::cuda::CUDAGuard guard(q.device());
  if (has(qt_seq)) {
    TORCH_CHECK(dtype == 1 && has(qt_start), "masked_attention: the tensor-core kernel takes bf16");
    check(lbk_masked_attention_mma(q.data_ptr(), q.stride(0), kmat.data_ptr(), vmat.data_ptr(), kmat.stride(0), meta(ext_off), meta(nsink),
                                   meta(cstart), ptr_opt(gate), ldg, meta(*qt_seq), meta(*qt_start), (int)qt_seq->numel(), meta(seq_off),
                                   meta(past), y.data_ptr(), y.stride(0), (int)H, (int)G, (int)D, (int)V, (int)window, (int)chunk, (int)keep,
                                   (float)scale, (float)softcap, (int)sink, (int)gate_wide, (float)out_scale, cur_stream()),
          "masked_attention (tensor cores)");
    return;
  }
  check(lbk_masked_attention(q.data_ptr(), q.stride(0), kmat.data_ptr(), vmat.data_ptr(), kmat.stride(0), nullptr, nullptr, 0, 0,
                             meta(ext_off), meta(nsink), meta(cstart), nullptr, ptr_opt(gate), ldg, meta(tok_seq), meta(seq_off), meta(past),
                             y.data_ptr(), y.stride(0), q.size(0), (int)H, (int)G, (int)D, (int)V, (int)window, (int)chunk, (int)keep,
                             (float)scale, (float)softcap, (int)sink, (int)gate_wide, (float)out_scale, dtype, cur_stream()), "masked_attention");
}

// single-token steps: keys / values straight from the ring and the kept-first rows.  splits == 0: one warp per (token, head);
// splits > 0: the grouped kernel, the keys of a (sequence, key head) cut into `splits` parts and merged.
void ring_attention(const Tensor& q, const Tensor& ring, const Tensor& first, const OptT& gate, const Tensor& tok_seq, const Tensor& seq_off,
                    const Tensor& slots, const Tensor& past, Tensor y, int64_t H, int64_t G, int64_t D, int64_t V, int64_t window,
                    int64_t chunk, int64_t keep, double scale, int64_t splits, double softcap, bool sink, bool gate_wide, double out_scale) {
  rows2d(q, "ring_attention q"); rows2d(y, "ring_attention y");
  const int dtype = code(q);
  ring_shapes(ring, first, G * (D + V));
  TORCH_CHECK(q.size(1) == H * D && y.size(1) == H * V && y.size(0) == q.size(0) && code(ring) == dtype && code(y) == dtype &&
              q.size(0) == slots.numel(), "ring_attention: shapes (one token per sequence)");
  long ldg = 0;
  if (has(gate)) { rows2d(*gate, "ring_attention gate"); TORCH_CHECK(gate->size(1) == (gate_wide ? H * V : H) && code(*gate) == dtype, "ring_attention: gate [tokens, H] (or [tokens, H V])"); ldg = gate->stride(0); }
  c10::cuda::CUDAGuard guard(q.device());
  if (splits > 0) {
    Tensor part = at::empty({q.size(0) * H * splits * (V + 2)}, q.options().dtype(at::kFloat));
    check(lbk_ring_decode(q.data_ptr(), q.stride(0), ring.data_ptr(), first.data_ptr(), (int)ring.size(1), (int)first.size(1), meta(slots),
                          meta(past), ptr_opt(gate), ldg, y.data_ptr(), y.stride(0), part.data_ptr<float>(), (int)q.size(0), (int)H, (int)G,
                          (int)D, (int)V, (int)window, (int)chunk, (int)keep, (float)scale, (int)splits, (float)softcap, (int)sink, (int)gate_wide,
                          (float)out_scale, dtype, cur_stream()), "ring_decode");
    return;
  }
  check(lbk_masked_attention(q.data_ptr(), q.stride(0), nullptr, nullptr, 0, ring.data_ptr(), first.data_ptr(), (int)ring.size(1),
                             (int)first.size(1), nullptr, nullptr, nullptr, meta(slots), ptr_opt(gate), ldg, meta(tok_seq), meta(seq_off),
                             meta(past), y.data_ptr(), y.stride(0), q.size(0), (int)H, (int)G, (int)D, (int)V, (int)window, (int)chunk,
                             (int)keep, (float)scale, (float)softcap, (int)sink, (int)gate_wide, (float)out_scale, dtype, cur_stream()),
        "ring_attention");
}

void moe_topk(const Tensor& z, const OptT& bias, int64_t mode, int64_t top, double rscale, Tensor idx, Tensor wts, const OptT& counts) {
  rows2d(z, "moe_topk z");
  TORCH_CHECK(z.scalar_type() == at::kFloat, "moe_topk: fp32 router logits expected");
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kInt && idx.is_contiguous() && idx.numel() == z.size(0) * top, "moe_topk: idx int32 [tokens, top]");
  TORCH_CHECK(wts.is_cuda() && wts.scalar_type() == at::kFloat && wts.is_contiguous() && wts.numel() == z.size(0) * top, "moe_topk: weights fp32 [tokens, top]");
  const float* bp = nullptr;
  if (has(bias)) { TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kFloat && bias->is_contiguous() && bias->numel() == z.size(1), "moe_topk: bias fp32 [E]"); bp = bias->data_ptr<float>(); }
  TORCH_CHECK(mode >= 0 && mode <= 2, "moe_topk: mode 0 (sigmoid scores, normalised), 1 (softmax over the chosen logits) or 2 (sigmoid scores as they are)");
  int* cp = nullptr;
  if (has(counts)) { TORCH_CHECK(counts->is_cuda() && counts->scalar_type() == at::kInt && counts->numel() >= z.size(1), "moe_topk: counts"); cp = counts->data_ptr<int>(); }
  c10::cuda::CUDAGuard guard(z.device());
  check(lbk_moe_topk(z.data_ptr<float>(), z.stride(0), bp, (int)mode, (int)z.size(1), (int)top, (float)rscale, idx.data_ptr<int>(), wts.data_ptr<float>(), cp,
                     z.size(0), cur_stream()), "moe_topk");
}

void moe_pairs(const Tensor& h, const Tensor& wgu, const Tensor& wd, const Tensor& idx, const Tensor& wts, Tensor a, Tensor out, int64_t act,
               double limit, bool weight_input) {
  rows2d(h, "moe_pairs h");
  const int64_t n = h.size(1), tokens = h.size(0), top = idx.numel() / std::max<int64_t>(tokens, 1);
  TORCH_CHECK(wgu.is_cuda() && wgu.dim() == 3 && wgu.is_contiguous() && wgu.size(2) == n && wgu.size(1) % 2 == 0 && code(wgu) == code(h), "moe_pairs: wgu [E, 2 ff, width]");
  const int64_t ff = wgu.size(1) / 2;
  TORCH_CHECK(wd.is_cuda() && wd.dim() == 3 && wd.is_contiguous() && wd.size(0) == wgu.size(0) && wd.size(1) == n && wd.size(2) == ff && code(wd) == code(h), "moe_pairs: wd [E, width, ff]");
  TORCH_CHECK(a.is_cuda() && a.is_contiguous() && a.numel() == tokens * top * ff && code(a) == code(h), "moe_pairs: a [tokens*top, ff]");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.is_contiguous() && out.numel() == tokens * n, "moe_pairs: out fp32 [tokens, width]");
  TORCH_CHECK(wts.scalar_type() == at::kFloat && wts.is_contiguous() && wts.numel() == idx.numel(), "moe_pairs: weights");
  c10::cuda::CUDAGuard guard(h.device());
  check(lbk_moe_pairs(h.data_ptr(), h.stride(0), wgu.data_ptr(), wd.data_ptr(), meta(idx), wts.data_ptr<float>(), a.data_ptr(), out.data_ptr<float>(),
                      tokens, (int)ff, (int)n, (int)top, (int)act, (float)limit, weight_input ? 1 : 0, code(h), cur_stream()), "moe_pairs");
}

// rows sorted by expert; with `tile_group` (int32 [rows of xs / align]) every expert's range starts on a multiple of `align`
void moe_sort(const Tensor& h, const Tensor& idx, const Tensor& counts, Tensor offsets, Tensor cursor, Tensor pos, Tensor xs, int64_t align,
              const OptT& tile_group, const OptT& wts) {
  rows2d(h, "moe_sort h");
  const float* wp = nullptr;
  if (has(wts)) {
    TORCH_CHECK(wts->is_cuda() && wts->scalar_type() == at::kFloat && wts->is_contiguous() && wts->numel() == idx.numel(), "moe_sort: weights fp32 [tokens, top]");
    wp = wts->data_ptr<float>();
  }
  const int64_t tokens = h.size(0), n = h.size(1), top = idx.numel() / std::max<int64_t>(tokens, 1), E = counts.numel();
  TORCH_CHECK(offsets.numel() == E + 1 && cursor.numel() >= E && pos.numel() == idx.numel(), "moe_sort: metadata sizes");
  TORCH_CHECK(xs.is_cuda() && xs.dim() == 2 && xs.is_contiguous() && xs.size(1) == n && code(xs) == code(h) &&
              xs.size(0) >= tokens * top + E * (align - 1), "moe_sort: xs [tokens*top (+ padding), width]");
  int* tg = nullptr; int tiles = 0;
  if (has(tile_group)) {
    TORCH_CHECK(align > 1 && xs.size(0) % align == 0 && tile_group->numel() == xs.size(0) / align, "moe_sort: one group entry per aligned block of xs");
    tg = const_cast<int*>(meta(*tile_group)); tiles = (int)tile_group->numel();
  }
  c10::cuda::CUDAGuard guard(h.device());
  check(lbk_moe_sort(h.data_ptr(), h.stride(0), meta(idx), meta(counts), const_cast<int*>(meta(offsets)), const_cast<int*>(meta(cursor)),
                     const_cast<int*>(meta(pos)), xs.data_ptr(), tokens, (int)E, (int)n, (int)top, (int)align, tg, tiles, wp, code(h), cur_stream()),
        "moe_sort");
}

// x fp32 [rows, n]: out = rmsnorm(alpha x + y1 + y2') (1 + w) into xout (fp32, may be x) and h (the model's dtype)
void postnorm_residual(const Tensor& x, const OptT& xout, const OptT& y1, const OptT& y2, const OptT& pos, const OptT& cw, double alpha,
                       const Tensor& w, double eps, const OptT& h) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && x.scalar_type() == at::kFloat, "postnorm_residual: x fp32 [rows, width]");
  const int64_t rows = x.size(0), n = x.size(1);
  const int dtype = code(w);
  TORCH_CHECK(w.is_cuda() && w.is_contiguous() && w.numel() == n, "postnorm_residual: weight [width]");
  float* xo = nullptr;
  if (has(xout)) {
    TORCH_CHECK(xout->is_cuda() && xout->is_contiguous() && xout->scalar_type() == at::kFloat && xout->numel() == x.numel(), "postnorm_residual: xout fp32 [rows, width]");
    xo = xout->data_ptr<float>();
  }
  const void* y1p = nullptr; long ldy1 = 0; int y1d = 0;
  if (has(y1)) {
    rows2d(*y1, "postnorm_residual y1");
    TORCH_CHECK(y1->size(0) == rows && y1->size(1) == n, "postnorm_residual: y1 [rows, width]");
    y1p = y1->data_ptr(); ldy1 = y1->stride(0); y1d = code(*y1);
  }
  const float* y2p = nullptr; long ldy2 = 0; const int* pp = nullptr; const float* cp = nullptr; int top = 0;
  if (has(y2)) {
    rows2d(*y2, "postnorm_residual y2");
    TORCH_CHECK(y2->scalar_type() == at::kFloat && y2->size(1) == n, "postnorm_residual: y2 fp32 [*, width]");
    y2p = y2->data_ptr<float>(); ldy2 = y2->stride(0);
    if (has(pos)) {
      TORCH_CHECK(pos->numel() % std::max<int64_t>(rows, 1) == 0, "postnorm_residual: pos [rows, top]");
      pp = meta(*pos); top = (int)(pos->numel() / std::max<int64_t>(rows, 1));
      if (has(cw)) {
        TORCH_CHECK(cw->is_cuda() && cw->scalar_type() == at::kFloat && cw->is_contiguous() && cw->numel() == pos->numel(), "postnorm_residual: cw fp32 [rows, top]");
        cp = cw->data_ptr<float>();
      }
    } else {
      TORCH_CHECK(y2->size(0) == rows, "postnorm_residual: y2 rows");
    }
  }
  void* hp = nullptr; long ldh = 0;
  if (has(h)) {
    rows2d(*h, "postnorm_residual h");
    TORCH_CHECK(h->size(0) == rows && h->size(1) == n && code(*h) == dtype, "postnorm_residual: h [rows, width] of the weight's dtype");
    hp = h->data_ptr(); ldh = h->stride(0);
  }
  c10::cuda::CUDAGuard guard(x.device());
  check(lbp_postnorm_residual(x.data_ptr<float>(), xo, y1p, ldy1, y1d, y2p, ldy2, pp, cp, top, (float)alpha, w.data_ptr(), (float)eps, hp, ldh,
                              rows, (int)n, dtype, cur_stream()), "postnorm_residual");
}

// q, k, v: column slices of one projection output (one row stride).  tail [slots, taps-1, H*D + G*D + G*V]; pool
// [pages, page_size, G*D + G*V]; table int32 [slots, max_pages]
void conv_qkv_prepare(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& wq, const Tensor& wk, const Tensor& wv, Tensor tail,
                      const Tensor& qn, const Tensor& kn, const Tensor& freq, double eps, Tensor qout, Tensor pool, const Tensor& table,
                      const Tensor& tok_seq, const Tensor& seq_off, const Tensor& slots, const Tensor& past, int64_t H, int64_t G, int64_t D,
                      int64_t V) {
  rows2d(q, "conv_qkv_prepare q"); rows2d(k, "conv_qkv_prepare k"); rows2d(v, "conv_qkv_prepare v"); rows2d(qout, "conv_qkv_prepare qout");
  const int dtype = code(q);
  const int64_t tokens = q.size(0), C = H * D + G * D + G * V;
  TORCH_CHECK(q.size(1) == H * D && k.size(1) == G * D && v.size(1) == G * V && k.size(0) == tokens && v.size(0) == tokens &&
              q.stride(0) == k.stride(0) && q.stride(0) == v.stride(0) && code(k) == dtype && code(v) == dtype, "conv_qkv_prepare: q, k, v slices of one matrix");
  TORCH_CHECK(wq.dim() == 2 && wq.is_contiguous() && wq.size(0) == H * D && wk.is_contiguous() && wk.size(0) == G * D && wv.is_contiguous() &&
              wv.size(0) == G * V && wk.size(1) == wq.size(1) && wv.size(1) == wq.size(1) && code(wq) == dtype && code(wk) == dtype &&
              code(wv) == dtype && wq.is_cuda() && wk.is_cuda() && wv.is_cuda(), "conv_qkv_prepare: convolution weights [channels, taps]");
  const int64_t taps = wq.size(1);
  TORCH_CHECK(tail.is_cuda() && tail.is_contiguous() && tail.dim() == 3 && tail.size(1) == taps - 1 && tail.size(2) == C && code(tail) == dtype,
              "conv_qkv_prepare: tail [slots, taps-1, channels]");
  vec(qn, D, dtype, "conv_qkv_prepare q norm"); vec(kn, D, dtype, "conv_qkv_prepare k norm");
  TORCH_CHECK(freq.is_cuda() && freq.scalar_type() == at::kFloat && freq.is_contiguous() && 2 * freq.numel() <= D, "conv_qkv_prepare: freq fp32 [rot/2]");
  TORCH_CHECK(qout.size(0) == tokens && qout.size(1) == H * D && code(qout) == dtype, "conv_qkv_prepare: qout [tokens, H*D]");
  TORCH_CHECK(pool.is_cuda() && pool.is_contiguous() && pool.dim() == 3 && pool.size(2) == G * D + G * V && code(pool) == dtype, "conv_qkv_prepare: pool [pages, page_size, G*D + G*V]");
  TORCH_CHECK(table.dim() == 2, "conv_qkv_prepare: table [slots, max_pages]");
  c10::cuda::CUDAGuard guard(q.device());
  check(lbp_conv_qkv_prepare(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), wq.data_ptr(), wk.data_ptr(), wv.data_ptr(), (int)taps,
                             tail.data_ptr(), qn.data_ptr(), kn.data_ptr(), freq.data_ptr<float>(), (int)freq.numel(), (float)eps, qout.data_ptr(),
                             qout.stride(0), pool.data_ptr(), meta(table), (int)table.size(1), (int)pool.size(1), meta(tok_seq), meta(seq_off),
                             meta(slots), meta(past), tokens, (int)slots.numel(), (int)H, (int)G, (int)D, (int)V, dtype, cur_stream()),
        "conv_qkv_prepare");
}

std::vector<int64_t> talk_attention_tiles(int64_t qt_max, int64_t H, int64_t G, int64_t D, int64_t V) {
  int kt = 0;
  const int qt = lbp_talk_attention_tiles((int)qt_max, (int)H, (int)G, (int)D, (int)V, &kt);
  return {qt, kt};
}

void talk_attention(const Tensor& q, const Tensor& pool, const Tensor& table, const OptT& talk, const OptT& sink, const Tensor& qt_seq,
                    const OptT& qt_start, int64_t QT, int64_t KT, const Tensor& seq_off, const Tensor& slots, const Tensor& past, Tensor y,
                    const OptT& part, int64_t nparts, int64_t H, int64_t G, int64_t D, int64_t V, double scale, double out_scale) {
  rows2d(q, "talk_attention q"); rows2d(y, "talk_attention y");
  const int dtype = code(q);
  const int64_t rows = q.size(0);
  TORCH_CHECK(q.size(1) == H * D && y.size(0) == rows && y.size(1) == H * V && code(y) == dtype, "talk_attention: q [rows, H*D], y [rows, H*V]");
  TORCH_CHECK(pool.is_cuda() && pool.is_contiguous() && pool.dim() == 3 && pool.size(2) == G * D + G * V && code(pool) == dtype, "talk_attention: pool [pages, page_size, G*D + G*V]");
  TORCH_CHECK(table.dim() == 2 && QT >= 1 && KT >= 1, "talk_attention: table [slots, max_pages]");
  const float* tp = nullptr; const float* sp = nullptr; float* pp = nullptr;
  if (has(talk)) { TORCH_CHECK(talk->is_cuda() && talk->scalar_type() == at::kFloat && talk->is_contiguous() && talk->numel() == H * H, "talk_attention: talk fp32 [H, H]"); tp = talk->data_ptr<float>(); }
  if (has(sink)) { TORCH_CHECK(sink->is_cuda() && sink->scalar_type() == at::kFloat && sink->is_contiguous() && sink->numel() == H, "talk_attention: sink fp32 [H]"); sp = sink->data_ptr<float>(); }
  if (QT == 16) {                               // the tensor-core prompt tiling (bf16; the launcher refuses sizes it is not built for)
    TORCH_CHECK(dtype == 1 && nparts == 1, "talk_attention: tiles of 16 queries are the bf16 tensor-core form");
    c10::cuda::CUDAGuard guard(q.device());
    check(lbp_talk_attention_mma(q.data_ptr(), q.stride(0), pool.data_ptr(), meta(table), (int)table.size(1), (int)pool.size(1), tp, sp,
                                 meta(qt_seq), meta_opt(qt_start), (int)qt_seq.numel(), meta(seq_off), meta(slots), meta(past), y.data_ptr(),
                                 y.stride(0), (int)H, (int)G, (int)D, (int)V, (float)scale, (float)out_scale, cur_stream()),
          "talk_attention (tensor cores)");
    return;
  }
  if (nparts > 1) {
    TORCH_CHECK(has(part) && part->is_cuda() && part->scalar_type() == at::kFloat && part->is_contiguous() && part->numel() >= rows * nparts * H * (V + 2), "talk_attention: part fp32 [rows, nparts, H, V + 2]");
    pp = part->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(q.device());
  check(lbp_talk_attention(q.data_ptr(), q.stride(0), pool.data_ptr(), meta(table), (int)table.size(1), (int)pool.size(1), tp, sp, meta(qt_seq),
                           meta_opt(qt_start), (int)qt_seq.numel(), (int)QT, (int)KT, meta(seq_off), meta(slots), meta(past), y.data_ptr(), y.stride(0),
                           pp, (int)nparts, rows, (int)H, (int)G, (int)D, (int)V, (float)scale, (float)out_scale, dtype, cur_stream()),
        "talk_attention");
}

}  // namespace

TORCH_LIBRARY(libai_b200_kv, m) {
  m.def("embed_scale(Tensor table, Tensor ids, float scale, Tensor(a!) x) -> ()", &embed_scale);
  m.def("dyt_residual(Tensor(a!) x, Tensor? y, Tensor? pos, Tensor? cw, Tensor? pw, Tensor? pb, Tensor? palpha, Tensor? nw, Tensor? nb, Tensor? nalpha, Tensor(b!)? h) -> ()", &dyt_residual);
  m.def("act_rows(Tensor inp, Tensor(a!) out, int act, bool gated, float limit=0.0) -> ()", &act_rows);
  m.def("softcap(Tensor(a!) l, float cap) -> ()", &softcap);
  m.def("qk_prepare(Tensor(a!) q, Tensor(b!)? k, Tensor? qw, Tensor? kw, Tensor freq, float mscale, int H, int G, int D, float eps, bool full_norm, bool unit_norm, Tensor tok_seq, Tensor seq_off, Tensor past) -> ()", &qk_prepare);
  m.def("kv_write(Tensor(a!) ring, Tensor(b!) first, Tensor knew, Tensor vnew, Tensor tok_seq, Tensor seq_off, Tensor slots, Tensor past) -> ()", &kv_write);
  m.def("kv_gather(Tensor ring, Tensor first, Tensor knew, Tensor vnew, Tensor ext_seq, Tensor ext_off, Tensor nsink, Tensor cstart, Tensor seq_off, Tensor slots, Tensor past, Tensor(a!) ext) -> ()", &kv_gather);
  m.def("masked_attention(Tensor q, Tensor kmat, Tensor vmat, Tensor ext_off, Tensor nsink, Tensor cstart, Tensor? gate, Tensor tok_seq, Tensor seq_off, Tensor past, Tensor? qt_seq, Tensor? qt_start, Tensor(a!) y, int H, int G, int D, int V, int window, int chunk, int keep, float scale, float softcap=0.0, bool sink=False, bool gate_wide=False, float out_scale=1.0) -> ()", &masked_attention);
  m.def("ring_attention(Tensor q, Tensor ring, Tensor first, Tensor? gate, Tensor tok_seq, Tensor seq_off, Tensor slots, Tensor past, Tensor(a!) y, int H, int G, int D, int V, int window, int chunk, int keep, float scale, int splits, float softcap=0.0, bool sink=False, bool gate_wide=False, float out_scale=1.0) -> ()", &ring_attention);
  m.def("moe_topk(Tensor z, Tensor? bias, int mode, int top, float rscale, Tensor(a!) idx, Tensor(b!) wts, Tensor(c!)? counts) -> ()", &moe_topk);
  m.def("moe_pairs(Tensor h, Tensor wgu, Tensor wd, Tensor idx, Tensor wts, Tensor(a!) a, Tensor(b!) out, int act, float limit=0.0, bool weight_input=False) -> ()", &moe_pairs);
  m.def("moe_sort(Tensor h, Tensor idx, Tensor counts, Tensor(a!) offsets, Tensor(b!) cursor, Tensor(c!) pos, Tensor(d!) xs, int align, Tensor(e!)? tile_group, Tensor? wts=None) -> ()", &moe_sort);
  m.def("postnorm_residual(Tensor x, Tensor(a!)? xout, Tensor? y1, Tensor? y2, Tensor? pos, Tensor? cw, float alpha, Tensor w, float eps, Tensor(b!)? h) -> ()", &postnorm_residual);
  m.def("conv_qkv_prepare(Tensor q, Tensor k, Tensor v, Tensor wq, Tensor wk, Tensor wv, Tensor(a!) tail, Tensor qn, Tensor kn, Tensor freq, float eps, Tensor(b!) qout, Tensor(c!) pool, Tensor table, Tensor tok_seq, Tensor seq_off, Tensor slots, Tensor past, int H, int G, int D, int V) -> ()", &conv_qkv_prepare);
  m.def("talk_attention_tiles(int qt_max, int H, int G, int D, int V) -> int[]", &talk_attention_tiles);
  m.def("talk_attention(Tensor q, Tensor pool, Tensor table, Tensor? talk, Tensor? sink, Tensor qt_seq, Tensor? qt_start, int QT, int KT, Tensor seq_off, Tensor slots, Tensor past, Tensor(a!) y, Tensor(b!)? part, int nparts, int H, int G, int D, int V, float scale, float out_scale) -> ()", &talk_attention);
}
