// torch.ops.libai_b200_seq.* : argument-checking wrappers around the launchers of seq_mixers.cu (ragged batches with
// per-sequence state).  A library of its own so that a model that only needs these kernels builds nothing else.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

extern "C" {
int lbs_rmsnorm(const void* x, long ldx, int xdtype, const int64_t* ids, const void* w, float offset, float eps, void* y, long ldy,
                int ydtype, int wdtype, long rows, int n, cudaStream_t s);
int lbs_slice_act(const void* in, long ldi, int idtype, void* out, long ldo, int odtype, long rows, int n, int act, cudaStream_t s);
int lbs_short_conv(const void* in, long ldi, const void* w, void* tail, const int* tok_seq, const int* seq_off, const int* slots,
                   const int* past, void* out, long ldo, long tokens, int B, int C, int taps, int dtype, cudaStream_t s);
int lbs_delta_scan(const void* qkv, long ldq, int koff, int voff, const void* a, long lda, const void* bl, long ldb, const void* A_log,
                   const void* dt_bias, float* S, const int* seq_off, const int* slots, const int* past, float* out, float* work,
                   long tokens, int B, int H, int KH, int D, int V, int chan, int dtype, cudaStream_t s);
int lbs_gated_rmsnorm(const float* o, const void* gate, long ldg, const void* w, float eps, int act, void* y, long ldy, long rows,
                      int H, int V, int dtype, cudaStream_t s);
int lbs_latent_gather(const void* ring, const void* cnew, const int* ext_seq, const int* ext_off, const int* seq_off, const int* slots,
                      const int* past, void* ext, long rows, int C, int ring_len, int dtype, cudaStream_t s);
int lbs_latent_write(void* ring, const void* cnew, const int* tok_seq, const int* seq_off, const int* slots, const int* past,
                     long tokens, int C, int ring_len, int dtype, cudaStream_t s);
int lbs_window_attention(const void* q, long ldq, const void* kv, long ldkv, const void* gate, long ldg, const int* tok_seq,
                         const int* seq_off, const int* ext_off, const int* qt_seq, const int* qt_start, int n_qtiles, void* y,
                         long ldy, long tokens, int H, int D, int V, int window, float scale, int dtype, cudaStream_t s);
int lbs_latent_decode(const float* qa, const void* ring, const void* cnew, const int* slots, const int* past, float* out,
                      float* part_o, float* part_ml, int B, int H, int C, int ring_len, int window, float scale, int dtype,
                      cudaStream_t s);
int lbs_head_gate(const float* x, const void* gate, long ldg, void* y, long ldy, long rows, int H, int V, int dtype, cudaStream_t s);
}

namespace {
using at::Tensor;

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

void rmsnorm(const Tensor& x, const c10::optional<Tensor>& ids, const Tensor& w, double offset, double eps, Tensor out) {
  rows2d(x, "rmsnorm x"); rows2d(out, "rmsnorm out");
  const int n = (int)x.size(1);
  TORCH_CHECK(w.numel() == n && w.is_contiguous() && out.size(1) == n, "rmsnorm: width mismatch");
  const int64_t* idp = nullptr;
  long rows = x.size(0);
  if (ids.has_value() && ids->defined()) {
    TORCH_CHECK(ids->is_cuda() && ids->scalar_type() == at::kLong && ids->is_contiguous(), "rmsnorm: int64 ids expected");
    idp = ids->data_ptr<int64_t>(); rows = ids->numel();
  }
  TORCH_CHECK(out.size(0) == rows, "rmsnorm: row mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  check(lbs_rmsnorm(x.data_ptr(), x.stride(0), code(x), idp, w.data_ptr(), (float)offset, (float)eps, out.data_ptr(), out.stride(0),
                    code(out), code(w), rows, n, cur_stream()), "rmsnorm");
}

void slice_act(const Tensor& in, Tensor out, int64_t act) {
  rows2d(in, "slice_act in"); rows2d(out, "slice_act out");
  TORCH_CHECK(in.sizes() == out.sizes(), "slice_act: shape mismatch");
  c10::cuda::CUDAGuard guard(in.device());
  check(lbs_slice_act(in.data_ptr(), in.stride(0), code(in), out.data_ptr(), out.stride(0), code(out), in.size(0), (int)in.size(1),
                      (int)act, cur_stream()), "slice_act");
}

void short_conv(const Tensor& in, const Tensor& w, Tensor tail, const Tensor& tok_seq, const Tensor& seq_off, const Tensor& slots,
                const Tensor& past, Tensor out) {
  rows2d(in, "short_conv in"); rows2d(out, "short_conv out");
  const int C = (int)in.size(1), taps = (int)w.size(1);
  TORCH_CHECK(w.dim() == 2 && w.size(0) == C && w.is_contiguous() && out.size(1) == C && out.size(0) == in.size(0), "short_conv: shapes");
  TORCH_CHECK(tail.dim() == 3 && tail.size(1) == taps - 1 && tail.size(2) == C && tail.is_contiguous(), "short_conv: tail [slots, taps-1, C]");
  TORCH_CHECK(code(in) == code(w) && code(in) == code(tail) && code(in) == code(out), "short_conv: one dtype expected");
  c10::cuda::CUDAGuard guard(in.device());
  check(lbs_short_conv(in.data_ptr(), in.stride(0), w.data_ptr(), tail.data_ptr(), meta(tok_seq), meta(seq_off), meta(slots), meta(past),
                       out.data_ptr(), out.stride(0), in.size(0), (int)slots.numel(), C, taps, code(in), cur_stream()), "short_conv");
}

void delta_scan(const Tensor& qkv, int64_t koff, int64_t voff, const Tensor& a, const Tensor& b, const Tensor& A_log,
                const Tensor& dt_bias, Tensor S, const Tensor& seq_off, const Tensor& slots, const Tensor& past, Tensor out,
                int64_t KH, bool chan) {
  rows2d(qkv, "delta_scan qkv"); rows2d(a, "delta_scan a"); rows2d(b, "delta_scan b");
  TORCH_CHECK(S.dim() == 4 && S.is_contiguous() && S.scalar_type() == at::kFloat, "delta_scan: S must be fp32 [slots, H, D, V]");
  const int H = (int)S.size(1), D = (int)S.size(2), V = (int)S.size(3);
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous() && out.dim() == 2 && out.size(1) == (long)H * V &&
              out.size(0) == qkv.size(0), "delta_scan: out must be fp32 [tokens, H*V]");
  TORCH_CHECK(b.size(1) == H && a.size(1) == (chan ? (long)H * D : (long)H) && A_log.numel() == H &&
              dt_bias.numel() == (chan ? (long)H * D : (long)H), "delta_scan: gate shapes");
  TORCH_CHECK(qkv.size(1) >= voff + (long)H * V && voff >= koff + KH * D && koff >= KH * D, "delta_scan: qkv layout");
  TORCH_CHECK(code(qkv) == code(a) && code(qkv) == code(b) && code(qkv) == code(A_log) && code(qkv) == code(dt_bias),
              "delta_scan: one dtype expected");
  TORCH_CHECK(A_log.is_contiguous() && dt_bias.is_contiguous(), "delta_scan: contiguous constants");
  c10::cuda::CUDAGuard guard(qkv.device());
  const int64_t tokens = qkv.size(0);
  Tensor work = at::empty({tokens * (2 * KH * D + KH + H + (chan ? (int64_t)H * D : (int64_t)H))}, out.options());
  check(lbs_delta_scan(qkv.data_ptr(), qkv.stride(0), (int)koff, (int)voff, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
                       A_log.data_ptr(), dt_bias.data_ptr(), S.data_ptr<float>(), meta(seq_off), meta(slots), meta(past),
                       out.data_ptr<float>(), work.data_ptr<float>(), tokens, (int)slots.numel(), H, (int)KH, D, V, chan ? 1 : 0, code(qkv), cur_stream()), "delta_scan");
}

void gated_rmsnorm(const Tensor& o, const Tensor& gate, const Tensor& w, double eps, int64_t act, Tensor y, int64_t H, int64_t V) {
  rows2d(gate, "gated_rmsnorm gate"); rows2d(y, "gated_rmsnorm y");
  TORCH_CHECK(o.scalar_type() == at::kFloat && o.is_contiguous() && o.numel() == y.size(0) * H * V, "gated_rmsnorm: o fp32 [rows, H*V]");
  TORCH_CHECK(gate.size(1) == H * V && y.size(1) == H * V && w.numel() == V && w.is_contiguous(), "gated_rmsnorm: shapes");
  TORCH_CHECK(code(gate) == code(w) && code(gate) == code(y), "gated_rmsnorm: one dtype expected");
  c10::cuda::CUDAGuard guard(o.device());
  check(lbs_gated_rmsnorm(o.data_ptr<float>(), gate.data_ptr(), gate.stride(0), w.data_ptr(), (float)eps, (int)act, y.data_ptr(),
                          y.stride(0), y.size(0), (int)H, (int)V, code(y), cur_stream()), "gated_rmsnorm");
}

void latent_gather(const Tensor& ring, const Tensor& cnew, const Tensor& ext_seq, const Tensor& ext_off, const Tensor& seq_off,
                   const Tensor& slots, const Tensor& past, Tensor ext) {
  TORCH_CHECK(ring.dim() == 3 && ring.is_contiguous() && cnew.dim() == 2 && cnew.is_contiguous() && ext.dim() == 2 && ext.is_contiguous(),
              "latent_gather: contiguous ring [slots, len, C], new [tokens, C], ext [rows, C]");
  const int C = (int)ring.size(2);
  TORCH_CHECK(cnew.size(1) == C && ext.size(1) == C && code(ring) == code(cnew) && code(ring) == code(ext), "latent_gather: shapes");
  c10::cuda::CUDAGuard guard(ring.device());
  check(lbs_latent_gather(ring.data_ptr(), cnew.data_ptr(), meta(ext_seq), meta(ext_off), meta(seq_off), meta(slots), meta(past),
                          ext.data_ptr(), ext.size(0), C, (int)ring.size(1), code(ring), cur_stream()), "latent_gather");
}

void latent_write(Tensor ring, const Tensor& cnew, const Tensor& tok_seq, const Tensor& seq_off, const Tensor& slots, const Tensor& past) {
  TORCH_CHECK(ring.dim() == 3 && ring.is_contiguous() && cnew.dim() == 2 && cnew.is_contiguous() && cnew.size(1) == ring.size(2) &&
              code(ring) == code(cnew), "latent_write: shapes");
  c10::cuda::CUDAGuard guard(ring.device());
  check(lbs_latent_write(ring.data_ptr(), cnew.data_ptr(), meta(tok_seq), meta(seq_off), meta(slots), meta(past), cnew.size(0),
                         (int)ring.size(2), (int)ring.size(1), code(ring), cur_stream()), "latent_write");
}

void window_attention(const Tensor& q, const Tensor& kv, const c10::optional<Tensor>& gate, const Tensor& tok_seq, const Tensor& seq_off,
                      const Tensor& ext_off, const c10::optional<Tensor>& qt_seq, const c10::optional<Tensor>& qt_start, Tensor y,
                      int64_t H, int64_t D, int64_t V, int64_t window, double scale) {
  rows2d(q, "window_attention q"); rows2d(kv, "window_attention kv"); rows2d(y, "window_attention y");
  TORCH_CHECK(q.size(1) == H * D && kv.size(1) == H * (D + V) && y.size(1) == H * V && y.size(0) == q.size(0), "window_attention: shapes");
  TORCH_CHECK(code(q) == code(kv) && code(q) == code(y), "window_attention: one dtype expected");
  const void* gp = nullptr; long ldg = 0;
  if (gate.has_value() && gate->defined()) {
    rows2d(*gate, "window_attention gate");
    TORCH_CHECK(gate->size(1) == H && gate->size(0) == q.size(0) && code(*gate) == code(q), "window_attention: gate [tokens, H]");
    gp = gate->data_ptr(); ldg = gate->stride(0);
  }
  const int *qs = nullptr, *qb = nullptr;
  int nq = 0;
  if (qt_seq.has_value() && qt_seq->defined() && qt_start.has_value() && qt_start->defined()) {
    qs = meta(*qt_seq); qb = meta(*qt_start); nq = (int)qt_seq->numel();
    TORCH_CHECK(qt_start->numel() == nq, "window_attention: query tile lists differ in length");
  }
  c10::cuda::CUDAGuard guard(q.device());
  check(lbs_window_attention(q.data_ptr(), q.stride(0), kv.data_ptr(), kv.stride(0), gp, ldg, meta(tok_seq), meta(seq_off), meta(ext_off),
                             qs, qb, nq, y.data_ptr(), y.stride(0), q.size(0), (int)H, (int)D, (int)V, (int)window, (float)scale, code(q),
                             cur_stream()), "window_attention");
}

void latent_decode(const Tensor& qa, const Tensor& ring, const Tensor& cnew, const Tensor& slots, const Tensor& past, Tensor out,
                   int64_t window, double scale) {
  TORCH_CHECK(qa.scalar_type() == at::kFloat && qa.is_contiguous() && qa.dim() == 3 && out.scalar_type() == at::kFloat &&
              out.is_contiguous() && out.sizes() == qa.sizes(), "latent_decode: qa / out fp32 [B, H, C]");
  TORCH_CHECK(ring.dim() == 3 && ring.is_contiguous() && cnew.dim() == 2 && cnew.is_contiguous() && ring.size(2) == qa.size(2) &&
              cnew.size(1) == qa.size(2) && cnew.size(0) == qa.size(0) && code(ring) == code(cnew), "latent_decode: shapes");
  TORCH_CHECK(ring.size(1) >= window, "latent_decode: the ring is shorter than the window");
  c10::cuda::CUDAGuard guard(qa.device());
  Tensor part_o, part_ml;
  float *po = nullptr, *pm = nullptr;
  if (window > 64) {                                  // long windows: partial softmax per 32 positions, merged afterwards
    const int64_t nch = (window + 31) / 32;
    part_o = at::empty({qa.size(0), qa.size(1), nch, qa.size(2)}, qa.options());
    part_ml = at::empty({qa.size(0), qa.size(1), nch, 2}, qa.options());
    po = part_o.data_ptr<float>(); pm = part_ml.data_ptr<float>();
  }
  check(lbs_latent_decode(qa.data_ptr<float>(), ring.data_ptr(), cnew.data_ptr(), meta(slots), meta(past), out.data_ptr<float>(),
                          po, pm, (int)qa.size(0), (int)qa.size(1), (int)qa.size(2), (int)ring.size(1), (int)window, (float)scale, code(ring),
                          cur_stream()), "latent_decode");
}

void head_gate(const Tensor& x, const c10::optional<Tensor>& gate, Tensor y, int64_t H, int64_t V) {
  rows2d(y, "head_gate y");
  TORCH_CHECK(x.scalar_type() == at::kFloat && x.is_contiguous() && x.numel() == y.size(0) * H * V && y.size(1) == H * V, "head_gate: shapes");
  const void* gp = nullptr; long ldg = 0;
  if (gate.has_value() && gate->defined()) {
    rows2d(*gate, "head_gate gate");
    TORCH_CHECK(gate->size(1) == H && code(*gate) == code(y), "head_gate: gate [rows, H]");
    gp = gate->data_ptr(); ldg = gate->stride(0);
  }
  c10::cuda::CUDAGuard guard(x.device());
  check(lbs_head_gate(x.data_ptr<float>(), gp, ldg, y.data_ptr(), y.stride(0), y.size(0), (int)H, (int)V, code(y), cur_stream()), "head_gate");
}
}  // namespace

TORCH_LIBRARY(libai_b200_seq, m) {
  m.def("rmsnorm(Tensor x, Tensor? ids, Tensor w, float offset, float eps, Tensor(a!) out) -> ()", &rmsnorm);
  m.def("slice_act(Tensor inp, Tensor(a!) out, int act) -> ()", &slice_act);
  m.def("short_conv(Tensor inp, Tensor w, Tensor(a!) tail, Tensor tok_seq, Tensor seq_off, Tensor slots, Tensor past, Tensor(b!) out) -> ()", &short_conv);
  m.def("delta_scan(Tensor qkv, int koff, int voff, Tensor a, Tensor b, Tensor A_log, Tensor dt_bias, Tensor(a!) S, Tensor seq_off, Tensor slots, Tensor past, Tensor(b!) out, int kv_heads, bool chan) -> ()", &delta_scan);
  m.def("gated_rmsnorm(Tensor o, Tensor gate, Tensor w, float eps, int act, Tensor(a!) y, int H, int V) -> ()", &gated_rmsnorm);
  m.def("latent_gather(Tensor ring, Tensor cnew, Tensor ext_seq, Tensor ext_off, Tensor seq_off, Tensor slots, Tensor past, Tensor(a!) ext) -> ()", &latent_gather);
  m.def("latent_write(Tensor(a!) ring, Tensor cnew, Tensor tok_seq, Tensor seq_off, Tensor slots, Tensor past) -> ()", &latent_write);
  m.def("window_attention(Tensor q, Tensor kv, Tensor? gate, Tensor tok_seq, Tensor seq_off, Tensor ext_off, Tensor? qt_seq, Tensor? qt_start, Tensor(a!) y, int H, int D, int V, int window, float scale) -> ()", &window_attention);
  m.def("latent_decode(Tensor qa, Tensor ring, Tensor cnew, Tensor slots, Tensor past, Tensor(a!) out, int window, float scale) -> ()", &latent_decode);
  m.def("head_gate(Tensor x, Tensor? gate, Tensor(a!) y, int H, int V) -> ()", &head_gate);
}
