// Torch operator boundary of the masked-attention group:
//
//   recsys_ops::mha_fwd_with_mask(Tensor q, Tensor k, Tensor v, Tensor mask) -> Tensor
//
// Same schema string, namespace, dispatch key and argument contract as the
// reference registration (csrc/fa/fa_bindings.cpp:23-47 with
// csrc/custom_ops_macros.h:65-135) and the same checks, in the same order and
// with the same messages, as its op layer (csrc/fa/fa_fwd_op.cu:53-108), so the
// reference's tests read unchanged against it.  The body allocates the output and
// the scratch with torch's caching allocator on q's device, then hands plain
// pointers to the C ABI (include/fa_mask_fwd_sm100.h) on the current stream.
//
// A second operator, which the reference does not have, returns the log-sum-exp of every row
// as well (natural log, fp32, (B, H, Sq); -inf for a fully masked row) - what a backward pass
// or a merge of partial results over key ranges needs:
//
//   recsys_ops::mha_fwd_with_mask_lse(Tensor q, Tensor k, Tensor v, Tensor mask) -> (Tensor, Tensor)
//
// A third one takes the mask as a rule instead of a tensor (causal, sliding window, valid
// lengths: the recipes of examples/custom_mask_demo.py:33-65) and evaluates it inside the kernel:
//
//   recsys_ops::mha_fwd_rule_mask(Tensor q, Tensor k, Tensor v, bool causal, int window,
//                                 Tensor? valid_lens) -> Tensor
//
// Differences from the reference, on purpose: K, V and the mask are never padded
// here -- ragged seqlen_k is handled inside the launcher -- and CPU tensors raise
// the same "only supported on CUDA" error the reference's CPU stub raises
// (csrc/fa/fa_fwd_op.cu:200-207).

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../../include/fa_mask_fwd_sm100.h"

namespace {

std::tuple<torch::Tensor, torch::Tensor> forward_cuda(const torch::Tensor& q, const torch::Tensor& k,
                                                      const torch::Tensor& v, const torch::Tensor& mask,
                                                      bool want_lse) {
    TORCH_CHECK(q.is_cuda(), "q must be a CUDA tensor");
    TORCH_CHECK(k.is_cuda(), "k must be a CUDA tensor");
    TORCH_CHECK(v.is_cuda(), "v must be a CUDA tensor");
    TORCH_CHECK(mask.is_cuda(), "mask must be a CUDA tensor");

    const bool is_fp16 = q.dtype() == torch::kHalf;
    const bool is_bf16 = q.dtype() == torch::kBFloat16;
    TORCH_CHECK(is_fp16 || is_bf16, "q must be float16 or bfloat16");
    const auto want = is_fp16 ? torch::kHalf : torch::kBFloat16;
    TORCH_CHECK(k.dtype() == want, "k dtype must match q");
    TORCH_CHECK(v.dtype() == want, "v dtype must match q");
    TORCH_CHECK(mask.dtype() == want, "mask dtype must match q");

    TORCH_CHECK(q.is_contiguous(), "q must be contiguous");
    TORCH_CHECK(k.is_contiguous(), "k must be contiguous");
    TORCH_CHECK(v.is_contiguous(), "v must be contiguous");
    TORCH_CHECK(mask.is_contiguous(), "mask must be contiguous");

    TORCH_CHECK(q.dim() == 4, "q must be 4D (B, H, Sq, d)");
    TORCH_CHECK(k.dim() == 4, "k must be 4D (B, Hk, Sk, d)");
    TORCH_CHECK(v.dim() == 4, "v must be 4D (B, Hk, Sk, d)");
    TORCH_CHECK(mask.dim() == 4, "mask must be 4D (B, 1, Sq, Sk)");

    const int64_t B = q.size(0), H = q.size(1), Sq = q.size(2), d = q.size(3);
    const int64_t Hk = k.size(1), Sk = k.size(2);
    TORCH_CHECK(k.size(0) == B && v.size(0) == B && mask.size(0) == B, "Batch size mismatch");
    TORCH_CHECK(k.size(3) == d && v.size(3) == d, "head_dim mismatch between q/k/v");
    TORCH_CHECK(v.size(1) == Hk && v.size(2) == Sk, "seqlen_k mismatch between k/v");
    TORCH_CHECK(Hk > 0 && H % Hk == 0, "n_heads must be divisible by n_kv_heads (GQA)");
    TORCH_CHECK(d == 64 || d == 128, "Only head_dim=64 or head_dim=128 is supported");
    TORCH_CHECK(mask.size(1) == 1 && mask.size(2) >= Sq && mask.size(3) >= Sk,
                "mask shape must be (B, 1, >=Sq, k-dim >= Sk)");
    TORCH_CHECK(k.device() == q.device() && v.device() == q.device() && mask.device() == q.device(),
                "q, k, v, mask must be on the same device");

    const c10::cuda::CUDAGuard guard(q.device());
    auto out = torch::empty_like(q);
    torch::Tensor lse;
    if (want_lse) lse = torch::empty({B, H, Sq}, q.options().dtype(torch::kFloat32));

    FaMaskFwdArgs a{};
    a.struct_size = sizeof(FaMaskFwdArgs);
    a.device = q.get_device();
    a.q = q.data_ptr();
    a.k = k.data_ptr();
    a.v = v.data_ptr();
    a.mask = mask.data_ptr();
    a.out = out.data_ptr();
    a.lse = want_lse ? lse.data_ptr<float>() : nullptr;
    a.batch = static_cast<int32_t>(B);
    a.heads = static_cast<int32_t>(H);
    a.heads_k = static_cast<int32_t>(Hk);
    a.seqlen_q = static_cast<int32_t>(Sq);
    a.seqlen_k = static_cast<int32_t>(Sk);
    a.head_dim = static_cast<int32_t>(d);
    a.mask_seqlen_q = static_cast<int32_t>(mask.size(2));
    a.mask_seqlen_k = static_cast<int32_t>(mask.size(3));
    a.mask_batch_stride = mask.stride(0);
    a.mask_row_stride = mask.stride(2);
    a.dtype = is_bf16 ? FA_SM100_BF16 : FA_SM100_FP16;
    a.num_splits = 0;
    a.out_fp32 = 0;

    size_t ws_bytes = 0;
    int rc = fa_mask_fwd_sm100_workspace_bytes(&a, &ws_bytes);
    TORCH_CHECK(rc == FA_SM100_OK, "mha_fwd_with_mask: ", fa_mask_fwd_sm100_strerror(rc));
    torch::Tensor ws;
    void* ws_ptr = nullptr;
    if (ws_bytes > 0) {
        ws = torch::empty({static_cast<int64_t>(ws_bytes)},
                          torch::TensorOptions().dtype(torch::kUInt8).device(q.device()));
        ws_ptr = ws.data_ptr();
    }
    auto stream = at::cuda::getCurrentCUDAStream(q.get_device());
    rc = fa_mask_fwd_sm100(&a, ws_ptr, ws_bytes, static_cast<void*>(stream.stream()));
    TORCH_CHECK(rc == FA_SM100_OK, "mha_fwd_with_mask: ", fa_mask_fwd_sm100_strerror(rc));
    return {out, lse};
}

torch::Tensor mha_fwd_with_mask_cuda(const torch::Tensor& q, const torch::Tensor& k,
                                     const torch::Tensor& v, const torch::Tensor& mask) {
    return std::get<0>(forward_cuda(q, k, v, mask, false));
}

torch::Tensor mha_fwd_with_mask_cpu(const torch::Tensor&, const torch::Tensor&,
                                    const torch::Tensor&, const torch::Tensor&) {
    TORCH_CHECK(false, "mha_fwd_with_mask is only supported on CUDA");
    return {};
}

torch::Tensor dispatch_mha_fwd_with_mask(const torch::Tensor& q, const torch::Tensor& k,
                                         const torch::Tensor& v, const torch::Tensor& mask) {
    return q.device().is_cuda() ? mha_fwd_with_mask_cuda(q, k, v, mask)
                                : mha_fwd_with_mask_cpu(q, k, v, mask);
}

torch::Tensor mha_fwd_rule_mask(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v,
                                bool causal, int64_t window, const c10::optional<torch::Tensor>& valid_lens) {
    TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda(), "mha_fwd_rule_mask is only supported on CUDA");
    const bool is_bf16 = q.dtype() == torch::kBFloat16;
    TORCH_CHECK(is_bf16 || q.dtype() == torch::kHalf, "q must be float16 or bfloat16");
    TORCH_CHECK(k.dtype() == q.dtype() && v.dtype() == q.dtype(), "k and v dtype must match q");
    TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous(), "q, k, v must be contiguous");
    TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "q must be (B, H, Sq, d), k and v (B, Hk, Sk, d)");
    const int64_t B = q.size(0), H = q.size(1), Sq = q.size(2), d = q.size(3);
    const int64_t Hk = k.size(1), Sk = k.size(2);
    TORCH_CHECK(k.size(0) == B && v.sizes() == k.sizes() && k.size(3) == d, "shape mismatch between q, k and v");
    TORCH_CHECK(Hk > 0 && H % Hk == 0, "n_heads must be divisible by n_kv_heads (GQA)");
    TORCH_CHECK(d == 64 || d == 128, "Only head_dim=64 or head_dim=128 is supported");
    TORCH_CHECK(window >= 0, "window must be >= 0");
    TORCH_CHECK(k.device() == q.device() && v.device() == q.device(), "q, k, v must be on the same device");
    const c10::cuda::CUDAGuard guard(q.device());
    torch::Tensor lens;
    if (valid_lens.has_value() && valid_lens->defined()) {
        TORCH_CHECK(valid_lens->numel() == B, "valid_lens must hold one length per batch element");
        lens = valid_lens->to(q.device(), torch::kInt32).contiguous();
    }
    auto out = torch::empty_like(q);
    auto ws = torch::empty({FA_SM100_RULE_WORKSPACE_BYTES}, torch::TensorOptions().dtype(torch::kUInt8).device(q.device()));
    FaMaskFwdArgs a{};
    a.struct_size = sizeof(FaMaskFwdArgs);
    a.device = q.get_device();
    a.q = q.data_ptr();
    a.k = k.data_ptr();
    a.v = v.data_ptr();
    a.out = out.data_ptr();
    a.batch = static_cast<int32_t>(B);
    a.heads = static_cast<int32_t>(H);
    a.heads_k = static_cast<int32_t>(Hk);
    a.seqlen_q = static_cast<int32_t>(Sq);
    a.seqlen_k = static_cast<int32_t>(Sk);
    a.head_dim = static_cast<int32_t>(d);
    a.dtype = is_bf16 ? FA_SM100_BF16 : FA_SM100_FP16;
    auto stream = at::cuda::getCurrentCUDAStream(q.get_device());
    const int rc = fa_mask_fwd_sm100_rule(&a, causal ? 1 : 0, static_cast<int32_t>(window),
                                          lens.defined() ? lens.data_ptr<int32_t>() : nullptr, ws.data_ptr(),
                                          FA_SM100_RULE_WORKSPACE_BYTES, static_cast<void*>(stream.stream()));
    TORCH_CHECK(rc == FA_SM100_OK, "mha_fwd_rule_mask: ", fa_mask_fwd_sm100_strerror(rc));
    return out;
}

std::tuple<torch::Tensor, torch::Tensor> dispatch_mha_fwd_with_mask_lse(const torch::Tensor& q,
                                                                        const torch::Tensor& k,
                                                                        const torch::Tensor& v,
                                                                        const torch::Tensor& mask) {
    TORCH_CHECK(q.device().is_cuda(), "mha_fwd_with_mask is only supported on CUDA");
    return forward_cuda(q, k, v, mask, true);
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(recsys_ops, m) {
    m.def("mha_fwd_with_mask(Tensor q, Tensor k, Tensor v, Tensor mask) -> Tensor");
    m.def("mha_fwd_with_mask_lse(Tensor q, Tensor k, Tensor v, Tensor mask) -> (Tensor, Tensor)");
    m.def("mha_fwd_rule_mask(Tensor q, Tensor k, Tensor v, bool causal, int window, Tensor? valid_lens) -> Tensor");
}

TORCH_LIBRARY_IMPL(recsys_ops, CompositeExplicitAutograd, m) {
    m.impl("mha_fwd_with_mask", &dispatch_mha_fwd_with_mask);
    m.impl("mha_fwd_with_mask_lse", &dispatch_mha_fwd_with_mask_lse);
    m.impl("mha_fwd_rule_mask", &mha_fwd_rule_mask);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "recsys_ops / FA group: mha_fwd_with_mask for sm_100a";
}
