// Torch C++ extension `mxmoe_ops`: the five operators of the reference's pybind module
// (mxmoe/kernels/src/ref_bind.cu:759-768 - gg_cutlass, gg_cutlass_share_fused, gg_mxmoe_share_fused,
// quant_inp_act, silu_mul_then_quant) with the same names, argument order and return tuples, as a thin layer
// over the C ABI of libmxmoe_b200.so (include/mxmoe_b200.h).  Torch supplies tensors, the caching allocator and the
// current stream; every kernel launch goes through the C ABI.  A failed call raises (TORCH_CHECK), as in the
// reference.  mxmoe_b200/ops.py is the same API in Python over ctypes (and has a few keyword-only extras).
#include <torch/extension.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cstring>
#include <tuple>
#include <vector>

#include "../../include/mxmoe_b200.h"

namespace {

using QP = std::tuple<int64_t, int64_t, int64_t, bool>;   // (a_bits, w_bits, gsize, sym), ref_bind.cu:33-36
using TensorList = std::vector<at::Tensor>;

void ok(int rc) { TORCH_CHECK(rc == MXMOE_OK, "mxmoe_b200 status ", rc, ": ", mxmoe_last_error()); }
void* stream_of(const at::Tensor& t) { return c10::cuda::getCurrentCUDAStream(t.get_device()).stream(); }
const void* ptr(const at::Tensor& t) { return t.defined() && t.numel() > 0 ? t.data_ptr() : nullptr; }

mxmoe_qparams to_q(const QP& q) {
  mxmoe_qparams o;
  std::memset(&o, 0, sizeof(o));
  o.a_bits = (int32_t)std::get<0>(q); o.w_bits = (int32_t)std::get<1>(q); o.gsize = (int32_t)std::get<2>(q);
  o.sym = std::get<3>(q) ? 1 : 0;
  return o;
}

// activation storage tag (ref_bind.cu:461-473): 0 fp16 copy, 1 int8 per token, 2 int4 per token
int act_tag(const QP& q) {
  const int64_t a = std::get<0>(q), g = std::get<2>(q);
  if (a >= 16) return 0;
  if (a == 8 && g == -1) return 1;
  if (a == 4 && g == -1) return 2;
  return -1;
}

// one grouped launch over a host list of problems; synchronises and checks like the reference launcher
void launch(std::vector<mxmoe_gg_problem>& probs, const at::Tensor& like) {
  if (probs.empty()) return;
  c10::cuda::CUDAGuard guard(like.device());
  const size_t bytes = mxmoe_gg_workspace_bytes((int)probs.size());
  at::Tensor ws = at::empty({(int64_t)bytes + 256}, like.options().dtype(at::kByte));
  void* base = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(ws.data_ptr()) + 255) & ~uintptr_t(255));
  void* st = stream_of(like);
  ok(mxmoe_gg_launch(probs.data(), (int)probs.size(), base, bytes, st));
  ok(mxmoe_gg_check(base, st));
}

mxmoe_gg_problem problem(const at::Tensor& A, const at::Tensor& B, const at::Tensor& C, int64_t M, int64_t N, int64_t K,
                         const mxmoe_qparams& q, const void* sa, const void* sb) {
  mxmoe_gg_problem p;
  std::memset(&p, 0, sizeof(p));
  p.A = A.data_ptr(); p.B = B.data_ptr(); p.C = C.data_ptr();
  p.scale_a = sa; p.scale_b = sb;
  p.M = (int32_t)M; p.N = (int32_t)N; p.K = (int32_t)K;
  p.q = q;
  return p;
}

// ref_bind.cu:312-431
TensorList gg_mxmoe_share_fused(TensorList inp, TensorList experts, TensorList scale_zp_a, TensorList scale_zp_b,
                                TensorList output, int64_t N, int64_t K, int64_t shared_N, int64_t shared_K,
                                std::vector<QP> qparams_per_exp, at::Tensor recv_tokens_per_exp, bool verbose) {
  const int64_t E = recv_tokens_per_exp.size(0);
  TORCH_CHECK(!inp.empty(), "inp must not be empty");
  TORCH_CHECK(recv_tokens_per_exp.device().is_cpu(), "recv_tokens_per_exp must be a CPU tensor");
  const int64_t num_tokens = inp.back().size(0);
  const bool has_shared = (int64_t)experts.size() > E;
  auto recv = recv_tokens_per_exp.to(at::kLong).contiguous();
  const int64_t* tokens = recv.data_ptr<int64_t>();
  std::vector<mxmoe_gg_problem> probs;
  size_t pidx = 0;
  for (int64_t e = 0; e < E + (has_shared ? 1 : 0); ++e) {
    const int64_t m = e == E ? num_tokens : tokens[e];
    if (m == 0) continue;
    TORCH_CHECK(pidx < inp.size(), "fewer inputs than non-empty experts");
    const int64_t n = e == E ? shared_N : N, k = e == E ? shared_K : K;
    const void* sa = pidx < scale_zp_a.size() ? ptr(scale_zp_a[pidx]) : nullptr;
    const void* sb = (size_t)e < scale_zp_b.size() ? ptr(scale_zp_b[e]) : nullptr;
    probs.push_back(problem(inp[pidx], experts[e], output[pidx], m, n, k, to_q(qparams_per_exp[e]), sa, sb));
    if (verbose) printf("problem %zu: [%ld,%ld,%ld]\n", pidx, (long)m, (long)n, (long)k);
    ++pidx;
  }
  TORCH_CHECK(pidx == inp.size(), inp.size(), " inputs for ", pidx, " non-empty experts");
  launch(probs, inp[0]);
  return output;
}

struct Routed {
  at::Tensor buffer, recv;   // rows gathered by expert, per-expert counts on the CPU
};
Routed route_fp16(const at::Tensor& inp, const at::Tensor& topk_ids, int64_t E, const c10::optional<at::Tensor>& inp_buffer,
                  const c10::optional<at::Tensor>& perm, const c10::optional<at::Tensor>& recv) {
  if (perm.has_value()) return {inp_buffer.value(), recv.value()};
  auto sorted = at::sort(topk_ids.reshape({-1}), /*stable=*/true, /*dim=*/0, /*descending=*/false);
  at::Tensor indices = std::get<1>(sorted).floor_divide(topk_ids.size(1));
  return {inp.index_select(0, indices), at::bincount(std::get<0>(sorted), {}, E).cpu()};
}

// ref_bind.cu:68-182: fp16 grouped GEMM (the reference runs CUTLASS GemmGrouped; here the fp16 scheme of the kernel)
at::Tensor gg_cutlass(at::Tensor inp, at::Tensor experts, at::Tensor topk_ids, at::Tensor output,
                      c10::optional<int64_t>, c10::optional<at::Tensor> inp_buffer_, c10::optional<at::Tensor> perm_indices_,
                      c10::optional<at::Tensor> recv_tokens_per_exp_) {
  TORCH_CHECK(inp.dim() == 2, "hidden must be 2D");
  TORCH_CHECK(inp.is_cuda() && experts.is_cuda(), "dev must be on cuda");
  const int64_t E = experts.size(0), N = experts.size(1), K = experts.size(2);
  Routed r = route_fp16(inp, topk_ids, E, inp_buffer_, perm_indices_, recv_tokens_per_exp_);
  auto recv = r.recv.to(at::kLong).contiguous();
  std::vector<mxmoe_gg_problem> probs;
  std::vector<at::Tensor> keep;
  const mxmoe_qparams q = to_q(QP{16, 16, -1, true});
  int64_t st = 0;
  for (int64_t e = 0; e < E; ++e) {
    const int64_t m = recv.data_ptr<int64_t>()[e];
    if (m == 0) continue;
    keep.push_back(r.buffer.narrow(0, st, m)); keep.push_back(output.narrow(0, st, m)); keep.push_back(experts[e]);
    probs.push_back(problem(keep[keep.size() - 3], keep.back(), keep[keep.size() - 2], m, N, K, q, nullptr, nullptr));
    st += m;
  }
  launch(probs, inp);
  return output;
}

// ref_bind.cu:184-310: routed experts plus the shared expert in one launch
std::tuple<at::Tensor, at::Tensor> gg_cutlass_share_fused(at::Tensor inp, at::Tensor experts, at::Tensor shared_experts,
                                                          at::Tensor topk_ids, at::Tensor output, at::Tensor shared_output,
                                                          c10::optional<int64_t>, c10::optional<at::Tensor> inp_buffer_,
                                                          c10::optional<at::Tensor> perm_indices_,
                                                          c10::optional<at::Tensor> recv_tokens_per_exp_) {
  TORCH_CHECK(inp.dim() == 2, "hidden must be 2D");
  TORCH_CHECK(inp.is_cuda() && experts.is_cuda(), "dev must be on cuda");
  const int64_t E = experts.size(0), N = experts.size(1), K = experts.size(2);
  Routed r = route_fp16(inp, topk_ids, E, inp_buffer_, perm_indices_, recv_tokens_per_exp_);
  auto recv = r.recv.to(at::kLong).contiguous();
  std::vector<mxmoe_gg_problem> probs;
  std::vector<at::Tensor> keep;
  const mxmoe_qparams q = to_q(QP{16, 16, -1, true});
  int64_t st = 0;
  for (int64_t e = 0; e < E; ++e) {
    const int64_t m = recv.data_ptr<int64_t>()[e];
    if (m == 0) continue;
    keep.push_back(r.buffer.narrow(0, st, m)); keep.push_back(output.narrow(0, st, m)); keep.push_back(experts[e]);
    probs.push_back(problem(keep[keep.size() - 3], keep.back(), keep[keep.size() - 2], m, N, K, q, nullptr, nullptr));
    st += m;
  }
  probs.push_back(problem(inp, shared_experts, shared_output, inp.size(0), shared_experts.size(0), shared_experts.size(1), q,
                          nullptr, nullptr));
  launch(probs, inp);
  return {output, shared_output};
}

// host tables of ref_bind.cu:475-505 / :636-668
struct Tables {
  std::vector<int32_t> tag, st, qoff, soff;
  std::vector<int64_t> qsize, ssize;
  int64_t q_total = 0, s_total = 0;
};
Tables expert_tables(const int64_t* tokens, int64_t num_tokens, int64_t E, bool has_shared, const std::vector<QP>& qp,
                     int64_t row_len, int64_t row_len_shared) {
  Tables t;
  int64_t acc = 0;
  for (int64_t e = 0; e < E + (has_shared ? 1 : 0); ++e) {
    const int tag = act_tag(qp[e]);
    TORCH_CHECK(tag >= 0, "activation scheme of expert ", e, " is not supported");
    const int64_t ld = e == E ? row_len_shared : row_len;
    const int64_t q_ld = tag == 0 ? ld : (tag == 1 ? ld / 2 : ld / 4);
    const int64_t m = e == E ? num_tokens : tokens[e];
    t.tag.push_back(tag); t.st.push_back((int32_t)acc); t.qoff.push_back((int32_t)t.q_total); t.soff.push_back((int32_t)t.s_total);
    t.qsize.push_back(q_ld * m); t.ssize.push_back(tag == 0 ? 0 : m);
    t.q_total += q_ld * m; t.s_total += tag == 0 ? 0 : m; acc += m;
  }
  return t;
}
at::Tensor tables_to_device(const Tables& t, const at::Tensor& like) {
  const int64_t n = (int64_t)t.tag.size();
  at::Tensor h = at::empty({4, n}, at::kInt);
  std::memcpy(h.data_ptr<int32_t>(), t.tag.data(), n * 4);
  std::memcpy(h.data_ptr<int32_t>() + n, t.st.data(), n * 4);
  std::memcpy(h.data_ptr<int32_t>() + 2 * n, t.qoff.data(), n * 4);
  std::memcpy(h.data_ptr<int32_t>() + 3 * n, t.soff.data(), n * 4);
  return h.to(like.device());
}
void fill_lists(const Tables& t, const int64_t* tokens, int64_t num_tokens, int64_t E, bool has_shared, int64_t row_len,
                int64_t row_len_shared, int64_t out_ld, int64_t out_ld_shared, const at::Tensor& q_store,
                const at::Tensor& s_store, const at::Tensor& out_store, TensorList& inp_list, TensorList& scale_list,
                TensorList& out_list) {
  int64_t out_off = 0;
  for (int64_t e = 0; e < E + (has_shared ? 1 : 0); ++e) {
    const int64_t m = e == E ? num_tokens : tokens[e];
    if (m == 0) continue;
    const int64_t ld = e == E ? row_len_shared : row_len;
    const int pack = t.tag[e] == 0 ? 1 : (t.tag[e] == 1 ? 2 : 4);
    inp_list.push_back(q_store.narrow(0, t.qoff[e], t.qsize[e]).view({m, ld / pack}));
    scale_list.push_back(t.s_total > 0 ? s_store.narrow(0, t.soff[e], t.ssize[e]) : at::empty({0}, q_store.options()));
    const int64_t old = e == E ? out_ld_shared : out_ld;
    out_list.push_back(out_store.narrow(0, out_off, m * old).view({m, old}));
    out_off += m * old;
  }
}

// ref_bind.cu:434-592
std::tuple<TensorList, TensorList, TensorList, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor>
quant_inp_act(at::Tensor hidden, at::Tensor topk_ids, int64_t num_experts, int64_t N, int64_t num_shared_experts,
              std::vector<QP> qparams_per_exp, bool verbose, bool rotate, c10::optional<at::Tensor> signs) {
  (void)verbose;
  TORCH_CHECK(hidden.dim() == 2 && hidden.is_cuda(), "hidden must be a 2D cuda tensor");
  TORCH_CHECK(hidden.scalar_type() == at::kHalf, "hidden must be fp16");
  TORCH_CHECK(topk_ids.scalar_type() == at::kInt, "topk_ids must be int32");
  c10::cuda::CUDAGuard guard(hidden.device());
  hidden = hidden.contiguous();
  const int64_t T = hidden.size(0), K = hidden.size(1), topk = topk_ids.size(1);
  const bool has_shared = num_shared_experts > 0;
  auto sorted = at::sort(topk_ids.reshape({-1}), /*stable=*/true, 0, false);
  at::Tensor dst_exp_sorted = std::get<0>(sorted);
  at::Tensor perm_indices = std::get<1>(sorted).floor_divide(topk);
  at::Tensor recv = at::bincount(dst_exp_sorted, {}, num_experts).cpu();
  const int64_t* tokens = recv.data_ptr<int64_t>();
  Tables tb = expert_tables(tokens, T, num_experts, has_shared, qparams_per_exp, K, K);
  at::Tensor tables = tables_to_device(tb, hidden);
  const int64_t n_all = (int64_t)tb.tag.size();
  auto f16 = hidden.options();
  at::Tensor inp_store = at::empty({tb.q_total}, f16), scale_store = at::empty({tb.s_total}, f16);
  at::Tensor out_store = at::empty({(num_shared_experts + topk) * T * N * 2}, f16);
  at::Tensor sg;
  if (signs.has_value()) sg = signs.value().to(hidden.device(), at::kChar).contiguous();

  // once per token into token-major stores, then one copy per routed row (same bits as one fused pass)
  bool used[3] = {false, false, false};
  for (int64_t e = 0; e < n_all; ++e)
    if ((e == num_experts ? T : tokens[e]) > 0) used[tb.tag[e]] = true;
  mxmoe_token_quant_args t;
  std::memset(&t, 0, sizeof(t));
  std::vector<at::Tensor> keep;
  auto store = [&](int64_t n) { keep.push_back(at::empty({n}, f16)); return keep.back().data_ptr(); };
  t.in = hidden.data_ptr(); t.k = (int32_t)K; t.num_tokens = (int32_t)T; t.rotate = rotate ? 1 : 0;
  t.signs = sg.defined() ? sg.data_ptr<int8_t>() : nullptr;
  if (used[0] && rotate) t.f16 = store(T * K);
  if (used[1]) { t.q8 = store(T * K / 2); t.s8 = store(T); }
  if (used[2]) { t.q4 = store(T * K / 4); t.s4 = store(T); }
  mxmoe_act_args a;
  std::memset(&a, 0, sizeof(a));
  const int32_t* tp = tables.data_ptr<int32_t>();
  a.q_store = inp_store.data_ptr(); a.s_store = tb.s_total ? scale_store.data_ptr() : nullptr;
  a.row_expert = dst_exp_sorted.data_ptr<int32_t>(); a.row_token = perm_indices.data_ptr<int64_t>();
  a.exp_qtag = tp; a.exp_row_start = tp + n_all; a.exp_q_off = tp + 2 * n_all; a.exp_s_off = tp + 3 * n_all;
  a.k = (int32_t)K; a.k_shared = (int32_t)K; a.rows_routed = (int32_t)(T * topk);
  a.rows_total = (int32_t)(T * topk + (has_shared ? T : 0)); a.num_experts = (int32_t)num_experts;
  a.rec_scale_off = -1;
  void* st = stream_of(hidden);
  ok(mxmoe_quant_tokens(&t, st));
  ok(mxmoe_gather_rows(&a, &t, st));
  for (auto& b : keep) b.record_stream(c10::cuda::getCurrentCUDAStream(hidden.get_device()));

  TensorList inp_list, scale_list, out_list;
  fill_lists(tb, tokens, T, num_experts, has_shared, K, K, N * 2, N * 2 * num_shared_experts, inp_store, scale_store,
             out_store, inp_list, scale_list, out_list);
  return {inp_list, scale_list, out_list, inp_store, scale_store, out_store, recv, perm_indices, dst_exp_sorted};
}

// ref_bind.cu:595-757
std::tuple<TensorList, TensorList, TensorList, at::Tensor, at::Tensor, at::Tensor>
silu_mul_then_quant(at::Tensor inp, int64_t num_problems, int64_t num_experts, int64_t K, int64_t N,
                    int64_t num_shared_experts, int64_t num_tokens, int64_t topk, at::Tensor values_sorted,
                    at::Tensor recv_tokens_per_exp, std::vector<QP> qparams_per_exp) {
  (void)num_problems;
  TORCH_CHECK(inp.is_cuda() && inp.scalar_type() == at::kHalf, "inp must be an fp16 cuda tensor");
  c10::cuda::CUDAGuard guard(inp.device());
  const bool has_shared = num_shared_experts > 0;
  auto recv = recv_tokens_per_exp.to(at::kLong).contiguous();
  const int64_t* tokens = recv.data_ptr<int64_t>();
  const int64_t n_shared = N * num_shared_experts;
  Tables tb = expert_tables(tokens, num_tokens, num_experts, has_shared, qparams_per_exp, N, n_shared);
  at::Tensor tables = tables_to_device(tb, inp);
  const int64_t n_all = (int64_t)tb.tag.size(), rows_routed = num_tokens * topk;
  auto f16 = inp.options();
  at::Tensor inp_store = at::empty({tb.q_total}, f16), scale_store = at::empty({tb.s_total}, f16);
  at::Tensor out_store = at::empty({(1 + topk) * num_tokens * K}, f16);
  at::Tensor flat = inp.reshape({-1});
  mxmoe_act_args a;
  std::memset(&a, 0, sizeof(a));
  const int32_t* tp = tables.data_ptr<int32_t>();
  a.in = flat.data_ptr();
  a.in_shared = has_shared ? static_cast<const void*>(static_cast<const at::Half*>(flat.data_ptr()) + rows_routed * N * 2) : nullptr;
  a.q_store = inp_store.data_ptr(); a.s_store = tb.s_total ? scale_store.data_ptr() : nullptr;
  a.row_expert = values_sorted.data_ptr<int32_t>();
  a.exp_qtag = tp; a.exp_row_start = tp + n_all; a.exp_q_off = tp + 2 * n_all; a.exp_s_off = tp + 3 * n_all;
  a.k = (int32_t)N; a.k_shared = (int32_t)(has_shared ? n_shared : N); a.rows_routed = (int32_t)rows_routed;
  a.rows_total = (int32_t)(rows_routed + (has_shared ? num_tokens : 0)); a.num_experts = (int32_t)num_experts;
  a.rec_scale_off = -1;
  ok(mxmoe_silu_mul_then_quant(&a, stream_of(inp)));
  TensorList inp_list, scale_list, out_list;
  fill_lists(tb, tokens, num_tokens, num_experts, has_shared, N, n_shared, K, K, inp_store, scale_store, out_store,
             inp_list, scale_list, out_list);
  return {inp_list, scale_list, out_list, inp_store, scale_store, out_store};
}

}  // namespace

PYBIND11_MODULE(mxmoe_ops, m) {
  m.doc() = "mxmoe_ops on the B200 kernels of libmxmoe_b200.so (operator API of mxmoe/kernels/src/ref_bind.cu:759-768)";
  namespace py = pybind11;
  m.def("gg_cutlass", &gg_cutlass, py::arg("inp"), py::arg("experts"), py::arg("topk_ids"), py::arg("output"),
        py::arg("num_problems_") = py::none(), py::arg("inp_buffer_") = py::none(), py::arg("perm_indices_") = py::none(),
        py::arg("recv_tokens_per_exp_") = py::none());
  m.def("gg_cutlass_share_fused", &gg_cutlass_share_fused, py::arg("inp"), py::arg("experts"), py::arg("shared_experts"),
        py::arg("topk_ids"), py::arg("output"), py::arg("shared_output"), py::arg("num_problems_") = py::none(),
        py::arg("inp_buffer_") = py::none(), py::arg("perm_indices_") = py::none(),
        py::arg("recv_tokens_per_exp_") = py::none());
  m.def("gg_mxmoe_share_fused", &gg_mxmoe_share_fused, py::arg("inp"), py::arg("experts"), py::arg("scale_zp_a"),
        py::arg("scale_zp_b"), py::arg("output"), py::arg("N"), py::arg("K"), py::arg("shared_N"), py::arg("shared_K"),
        py::arg("qparams_per_exp"), py::arg("recv_tokens_per_exp"), py::arg("verbose") = false);
  m.def("quant_inp_act", &quant_inp_act, py::arg("hidden"), py::arg("topk_ids"), py::arg("num_experts"), py::arg("N"),
        py::arg("num_shared_experts"), py::arg("qparams_per_exp"), py::arg("verbose") = false, py::arg("rotate") = false,
        py::arg("signs") = py::none());
  m.def("silu_mul_then_quant", &silu_mul_then_quant, py::arg("inp"), py::arg("num_problems"), py::arg("num_experts"),
        py::arg("K"), py::arg("N"), py::arg("num_shared_experts"), py::arg("num_tokens"), py::arg("topk"),
        py::arg("values_sorted"), py::arg("recv_tokens_per_exp"), py::arg("qparams_per_exp"));
}
