// torch.Tensor front end of the ring-attention forward.
//
// The reference's include/attention_api.cuh (lines 1-30) includes torch/extension.h and defines CHECK_CUDA /
// CHECK_CONTIGUOUS / CHECK_INPUT but declares no operator; this file is the operator those checks were written
// for.  Every function validates its tensors with CHECK_INPUT, takes the current torch CUDA stream, and calls the
// extern "C" entry points of ring_attention_b200.h.  Nothing is computed here and there is no fallback: a CPU
// tensor or a missing library is an error.  Forward only (the reference has no backward pass).
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <vector>

#include "../../include/attention_api.cuh"

namespace {

void check_qkv(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v) {
    CHECK_INPUT(q);
    CHECK_INPUT(k);
    CHECK_INPUT(v);
    TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q, k, v must be [batch, heads, rows, dim]");
    TORCH_CHECK(q.scalar_type() == at::kHalf || q.scalar_type() == at::kBFloat16, "q must be float16 or bfloat16");
    TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(), "q, k, v must share a dtype");
    TORCH_CHECK(k.sizes() == v.sizes(), "k and v must have the same shape");
    TORCH_CHECK(q.size(0) == k.size(0) && q.size(1) == k.size(1) && q.size(3) == k.size(3),
                "q and k must agree in batch, heads and dim");
    TORCH_CHECK(q.get_device() == k.get_device() && q.get_device() == v.get_device(), "q, k, v must be on one device");
}

void check_status(int status, const char* what) {
    TORCH_CHECK(status == RING_OK, what, " failed (", status, "): ", ring_last_error_string());
}

float default_scale(const at::Tensor& q, double softmax_scale) {
    return softmax_scale > 0.0 ? static_cast<float>(softmax_scale)
                               : 1.0f / std::sqrt(static_cast<float>(q.size(3)));
}

// One Q shard against one K/V shard (the flash inner loop of csrc/ring_attention.cu:536-609 plus :621-664).
std::vector<at::Tensor> block_forward(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double softmax_scale,
                                      bool causal, int64_t q_off, int64_t k_off) {
    check_qkv(q, k, v);
    const c10::cuda::CUDAGuard guard(q.device());
    auto out = at::empty(q.sizes(), q.options().dtype(at::kFloat));
    auto lse = at::empty({q.size(0), q.size(1), q.size(2)}, q.options().dtype(at::kFloat));
    check_status(ring_attention_block_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr<float>(),
                                          lse.data_ptr<float>(), static_cast<int>(q.size(0)), static_cast<int>(q.size(1)),
                                          static_cast<int>(q.size(2)), static_cast<int>(k.size(2)),
                                          static_cast<int>(q.size(3)), default_scale(q, softmax_scale), causal ? 1 : 0,
                                          q_off, k_off, /*merge=*/0, q.scalar_type() == at::kBFloat16 ? 1 : 0,
                                          at::cuda::getCurrentCUDAStream().stream()),
                 "ring_attention_block_fwd");
    return {out, lse};
}

// The ring forward of one rank (set_params_fprop + run_ring_fwd, csrc/ring_attention.cu:361-395, 669-704).
// `ctx` is the address of a RingCtx made by ring_ctx_create / ring_ctx_create_local; `seqlens` holds the rows of
// every rank's shard (the reference's seqlen[], :706).  Asynchronous on the current stream.
std::vector<at::Tensor> ring_forward(int64_t ctx, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                     std::vector<int64_t> seqlens, int64_t mype, double softmax_scale, bool causal) {
    check_qkv(q, k, v);
    TORCH_CHECK(ctx != 0, "ctx must be the address of a ring context");
    const int npes = static_cast<int>(seqlens.size());
    TORCH_CHECK(npes >= 1 && mype >= 0 && mype < npes, "mype must index seqlens");
    TORCH_CHECK(seqlens[mype] == q.size(2) && q.size(2) == k.size(2), "seqlens[mype] must equal the local rows of q and k");
    const c10::cuda::CUDAGuard guard(q.device());
    auto out = at::empty(q.sizes(), q.options().dtype(at::kFloat));
    auto lse = at::empty({q.size(0), q.size(1), q.size(2)}, q.options().dtype(at::kFloat));
    std::vector<int> h_seqlen(seqlens.begin(), seqlens.end());

    Ring_fwd_params params{};
    params.mype = static_cast<int>(mype);
    params.npes = npes;
    params.h_seqlen = h_seqlen.data();
    params.dim = static_cast<int>(q.size(3));
    params.softmax_scale = default_scale(q, softmax_scale);
    params.q_ptr = q.data_ptr();
    params.k_ptr = k.data_ptr();
    params.v_ptr = v.data_ptr();
    params.out_ptr = out.data_ptr<float>();
    params.batch = static_cast<int>(q.size(0));
    params.heads = static_cast<int>(q.size(1));
    params.lse_ptr = lse.data_ptr<float>();
    params.causal = causal ? 1 : 0;
    params.is_bf16 = q.scalar_type() == at::kBFloat16 ? 1 : 0;
    params.stream = at::cuda::getCurrentCUDAStream().stream();
    check_status(ring_attention_fwd(reinterpret_cast<RingCtx*>(ctx), &params), "ring_attention_fwd");
    return {out, lse};
}

// In-place merge of a partial result into the running one (csrc/ring_attention.cu:439-443, 597-598, 621-633).
void lse_merge_(at::Tensor& o_acc, at::Tensor& lse_acc, const at::Tensor& o_part, const at::Tensor& lse_part) {
    CHECK_INPUT(o_acc);
    CHECK_INPUT(lse_acc);
    CHECK_INPUT(o_part);
    CHECK_INPUT(lse_part);
    TORCH_CHECK(o_acc.scalar_type() == at::kFloat && lse_acc.scalar_type() == at::kFloat &&
                    o_part.scalar_type() == at::kFloat && lse_part.scalar_type() == at::kFloat,
                "merge operands must be float32");
    TORCH_CHECK(o_acc.sizes() == o_part.sizes() && lse_acc.sizes() == lse_part.sizes(), "merge operands must agree in shape");
    TORCH_CHECK(o_acc.dim() >= 2 && lse_acc.numel() * o_acc.size(-1) == o_acc.numel(), "lse must have one entry per row of o");
    const c10::cuda::CUDAGuard guard(o_acc.device());
    check_status(ring_lse_merge(o_acc.data_ptr<float>(), lse_acc.data_ptr<float>(), o_part.data_ptr<float>(),
                                lse_part.data_ptr<float>(), lse_acc.numel(), static_cast<int>(o_acc.size(-1)),
                                at::cuda::getCurrentCUDAStream().stream()),
                 "ring_lse_merge");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "torch.Tensor front end of the B200 ring-attention forward";
    m.def("block_forward", &block_forward, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("softmax_scale") = 0.0,
          py::arg("causal") = false, py::arg("q_off") = 0, py::arg("k_off") = 0,
          "Attention of one Q shard against one K/V shard: returns (out fp32, lse fp32)");
    m.def("ring_forward", &ring_forward, py::arg("ctx"), py::arg("q"), py::arg("k"), py::arg("v"), py::arg("seqlens"),
          py::arg("mype"), py::arg("softmax_scale") = 0.0, py::arg("causal") = false,
          "Ring-attention forward of rank mype: returns (out fp32, lse fp32)");
    m.def("lse_merge_", &lse_merge_, "Merge (o_part, lse_part) into (o_acc, lse_acc) in place");
}
