// PyTorch operator boundary of the sm_100a advantage library.
//
// Takes the place of both translation units of the reference extension
// `pufferlib._C`: pufferlib/extensions/pufferlib.cpp (module init :7-24, schema
// :87-89) and pufferlib/extensions/cuda/pufferlib.cu (argument checks :22-38,
// launcher :53-82, CUDA registration :84-86).  The operator namespace, name
// and schema string are the reference's, so
//   torch.ops.pufferlib.compute_puff_advantage(values, rewards, dones,
//       importance, advantages, gamma, lambda, rho_clip, c_clip)
// resolves here with pufferl.py:674 unchanged.  Only a CUDA kernel is
// registered: CPU tensors raise the dispatcher's "no kernel for backend" error
// instead of silently computing somewhere else.
//
// This file holds no arithmetic; it validates tensors, picks up the current
// device and stream, and calls the C ABI of include/puff_advantage.h.
#include <Python.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/all.h>
#include <torch/library.h>

#include <atomic>
#include <cstdlib>
#include <string>
#include <optional>
#include <tuple>

#include "../../include/puff_advantage.h"

extern "C" {
// Empty importable module: importing it loads this shared object, which runs
// the TORCH_LIBRARY registrations below (same device as pufferlib.cpp:7-24).
PyObject* PyInit__C(void)
{
    static struct PyModuleDef module_def = {PyModuleDef_HEAD_INIT, "_C", nullptr, -1, nullptr};
    return PyModule_Create(&module_def);
}
}

namespace pufferlib_b200 {

static void check_rc(int rc, const char* what)
{
    TORCH_CHECK(rc == PUFF_OK, what, ": ", puff_advantage_sm100_strerror(rc), " (code ", rc, ")");
}

// Same rules and messages as vtrace_check_cuda (cu:22-38), except that a
// non-contiguous tensor is an error: the reference calls t.contiguous() and
// drops the result (cu:34-36), then reads the strided storage as if dense.
static void check_inputs(std::initializer_list<torch::Tensor> tensors, const torch::Tensor& values)
{
    const auto device = values.device();
    const int64_t num_steps = values.dim() > 0 ? values.size(0) : 0;
    const int64_t horizon = values.dim() > 1 ? values.size(1) : 0;
    for (const torch::Tensor& t : tensors) {
        TORCH_CHECK(t.dim() == 2, "Tensor must be 2D");
        TORCH_CHECK(t.device() == device, "All tensors must be on same device");
        TORCH_CHECK(t.size(0) == num_steps, "First dimension must match num_steps");
        TORCH_CHECK(t.size(1) == horizon, "Second dimension must match horizon");
        TORCH_CHECK(t.dtype() == torch::kFloat32, "All tensors must be float32");
        TORCH_CHECK(t.is_contiguous(), "All tensors must be contiguous");
    }
    TORCH_CHECK(values.is_cuda(), "All tensors must be on GPU");
}

// Kernel variant of the three advantage ops: PUFF_VARIANT_AUTO unless the environment variable
// PUFFER_ADV_VARIANT (serial | scan | generic) said otherwise when the first op call was made, or
// puff_set_variant changed it since.  The op calls themselves read no environment.
static std::atomic<int>& variant_setting()
{
    static std::atomic<int> v{[] {
        const char* s = std::getenv("PUFFER_ADV_VARIANT");
        const std::string name(s == nullptr ? "" : s);
        return name == "serial" ? PUFF_VARIANT_SERIAL : name == "scan" ? PUFF_VARIANT_SCAN
             : name == "generic" ? PUFF_VARIANT_GENERIC : PUFF_VARIANT_AUTO;
    }()};
    return v;
}
static int variant_from_env() { return variant_setting().load(std::memory_order_relaxed); }

// puff_set_variant(v): v in PUFF_VARIANT_* ; returns the previous setting
int64_t puff_set_variant(int64_t v)
{
    TORCH_CHECK(v >= PUFF_VARIANT_AUTO && v <= PUFF_VARIANT_GENERIC, "unknown kernel variant");
    return variant_setting().exchange(static_cast<int>(v), std::memory_order_relaxed);
}

// compute_puff_advantage_cuda of cu:53-82
void compute_puff_advantage_cuda(torch::Tensor values, torch::Tensor rewards, torch::Tensor dones,
                                 torch::Tensor importance, torch::Tensor advantages, double gamma,
                                 double lambda, double rho_clip, double c_clip)
{
    check_inputs({values, rewards, dones, importance, advantages}, values);
    int rc;
    {
        const c10::cuda::CUDAGuard guard(values.device());
        rc = puff_advantage_sm100_launch(
            values.data_ptr<float>(), rewards.data_ptr<float>(), dones.data_ptr<float>(),
            importance.data_ptr<float>(), advantages.data_ptr<float>(), nullptr,
            static_cast<float>(gamma), static_cast<float>(lambda), static_cast<float>(rho_clip),
            static_cast<float>(c_clip), values.size(0), values.size(1), variant_from_env(),
            at::cuda::getCurrentCUDAStream().stream());
    }
    check_rc(rc, "compute_puff_advantage");
}

// Sibling op: the same launch with the fused epilogue.  seg_abs_sum[s] receives
// sum_t |advantages[s, t]| over t < H-1, what pufferl.py:359 computes with a
// second pass over a zero-initialised `advantages`.
void compute_puff_advantage_prio_cuda(torch::Tensor values, torch::Tensor rewards, torch::Tensor dones,
                                      torch::Tensor importance, torch::Tensor advantages,
                                      torch::Tensor seg_abs_sum, double gamma, double lambda,
                                      double rho_clip, double c_clip)
{
    check_inputs({values, rewards, dones, importance, advantages}, values);
    TORCH_CHECK(seg_abs_sum.dim() == 1 && seg_abs_sum.size(0) == values.size(0),
                "seg_abs_sum must be 1D with one entry per segment");
    TORCH_CHECK(seg_abs_sum.device() == values.device(), "All tensors must be on same device");
    TORCH_CHECK(seg_abs_sum.dtype() == torch::kFloat32, "All tensors must be float32");
    TORCH_CHECK(seg_abs_sum.is_contiguous(), "All tensors must be contiguous");
    int rc;
    {
        const c10::cuda::CUDAGuard guard(values.device());
        rc = puff_advantage_sm100_launch(
            values.data_ptr<float>(), rewards.data_ptr<float>(), dones.data_ptr<float>(),
            importance.data_ptr<float>(), advantages.data_ptr<float>(), seg_abs_sum.data_ptr<float>(),
            static_cast<float>(gamma), static_cast<float>(lambda), static_cast<float>(rho_clip),
            static_cast<float>(c_clip), values.size(0), values.size(1), variant_from_env(),
            at::cuda::getCurrentCUDAStream().stream());
    }
    check_rc(rc, "compute_puff_advantage_prio");
}

// The op with ownership of the whole output: also writes advantages[:, H-1] = 0,
// so the caller may pass torch.empty instead of the torch.zeros of pufferl.py:352-353.
// seg_abs_sum is optional.
void compute_puff_advantage_fill_cuda(torch::Tensor values, torch::Tensor rewards, torch::Tensor dones,
                                      torch::Tensor importance, torch::Tensor advantages,
                                      std::optional<torch::Tensor> seg_abs_sum, double gamma, double lambda,
                                      double rho_clip, double c_clip)
{
    check_inputs({values, rewards, dones, importance, advantages}, values);
    float* abs_ptr = nullptr;
    if (seg_abs_sum.has_value()) {
        const torch::Tensor& t = *seg_abs_sum;
        TORCH_CHECK(t.dim() == 1 && t.size(0) == values.size(0), "seg_abs_sum must be 1D with one entry per segment");
        TORCH_CHECK(t.device() == values.device(), "All tensors must be on same device");
        TORCH_CHECK(t.dtype() == torch::kFloat32, "All tensors must be float32");
        TORCH_CHECK(t.is_contiguous(), "All tensors must be contiguous");
        abs_ptr = t.data_ptr<float>();
    }
    int rc;
    {
        const c10::cuda::CUDAGuard guard(values.device());
        rc = puff_advantage_sm100_launch_ex(
            values.data_ptr<float>(), rewards.data_ptr<float>(), dones.data_ptr<float>(),
            importance.data_ptr<float>(), advantages.data_ptr<float>(), abs_ptr,
            static_cast<float>(gamma), static_cast<float>(lambda), static_cast<float>(rho_clip),
            static_cast<float>(c_clip), values.size(0), values.size(1), variant_from_env(),
            PUFF_FLAG_ZERO_LAST_COLUMN, at::cuda::getCurrentCUDAStream().stream());
    }
    check_rc(rc, "compute_puff_advantage_fill");
}

// pufferl.py:360 plus the sum of :361: weights and their fp64 total.
std::tuple<torch::Tensor, torch::Tensor> puff_priority_weights_cuda(torch::Tensor seg_abs_sum, double alpha)
{
    TORCH_CHECK(seg_abs_sum.is_cuda(), "All tensors must be on GPU");
    TORCH_CHECK(seg_abs_sum.dim() == 1 && seg_abs_sum.dtype() == torch::kFloat32 && seg_abs_sum.is_contiguous(),
                "seg_abs_sum must be a contiguous 1D float32 tensor");
    const c10::cuda::CUDAGuard guard(seg_abs_sum.device());
    const int64_t n = seg_abs_sum.size(0);
    auto weights = torch::empty_like(seg_abs_sum);
    auto total = torch::empty({1}, seg_abs_sum.options().dtype(torch::kFloat64));
    const size_t sbytes = puff_priorities_sm100_scratch_bytes(n);
    auto scratch = torch::empty({static_cast<int64_t>((sbytes + 7) / 8)}, seg_abs_sum.options().dtype(torch::kFloat64));
    const int rc = puff_priorities_sm100_weights(seg_abs_sum.data_ptr<float>(), weights.data_ptr<float>(),
                                                 total.data_ptr<double>(), static_cast<float>(alpha), n,
                                                 scratch.data_ptr<double>(), sbytes,
                                                 at::cuda::getCurrentCUDAStream().stream());
    check_rc(rc, "puff_priority_weights");
    return {weights, total};
}

// pufferl.py:361 given the (possibly all-reduced) total.
torch::Tensor puff_priority_probs_cuda(torch::Tensor weights, torch::Tensor total_w)
{
    TORCH_CHECK(weights.is_cuda() && total_w.is_cuda(), "All tensors must be on GPU");
    TORCH_CHECK(weights.dim() == 1 && weights.dtype() == torch::kFloat32 && weights.is_contiguous(),
                "weights must be a contiguous 1D float32 tensor");
    TORCH_CHECK(total_w.numel() == 1 && total_w.dtype() == torch::kFloat64, "total_w must hold one float64");
    const c10::cuda::CUDAGuard guard(weights.device());
    auto probs = torch::empty_like(weights);
    const int rc = puff_priorities_sm100_probs(weights.data_ptr<float>(), total_w.data_ptr<double>(),
                                               probs.data_ptr<float>(), weights.size(0),
                                               at::cuda::getCurrentCUDAStream().stream());
    check_rc(rc, "puff_priority_probs");
    return probs;
}

// The two priority steps of a sharded buffer with the exchange of the weight total done by the
// kernels (include/puff_advantage.h, puff_exchange).  `exchange` is the puff_exchange* as an integer.
torch::Tensor puff_priority_weights_push_cuda(torch::Tensor seg_abs_sum, double alpha, int64_t exchange)
{
    TORCH_CHECK(seg_abs_sum.is_cuda(), "All tensors must be on GPU");
    TORCH_CHECK(seg_abs_sum.dim() == 1 && seg_abs_sum.dtype() == torch::kFloat32 && seg_abs_sum.is_contiguous(),
                "seg_abs_sum must be a contiguous 1D float32 tensor");
    const c10::cuda::CUDAGuard guard(seg_abs_sum.device());
    const int64_t n = seg_abs_sum.size(0);
    auto weights = torch::empty_like(seg_abs_sum);
    const size_t sbytes = puff_priorities_sm100_scratch_bytes(n);
    auto scratch = torch::empty({static_cast<int64_t>((sbytes + 7) / 8)}, seg_abs_sum.options().dtype(torch::kFloat64));
    const int rc = puff_priorities_sm100_weights_push(seg_abs_sum.data_ptr<float>(), weights.data_ptr<float>(),
                                                      static_cast<float>(alpha), n, scratch.data_ptr<double>(), sbytes,
                                                      reinterpret_cast<puff_exchange*>(exchange),
                                                      at::cuda::getCurrentCUDAStream().stream());
    check_rc(rc, "puff_priority_weights_push");
    return weights;
}

std::tuple<torch::Tensor, torch::Tensor> puff_priority_probs_gathered_cuda(torch::Tensor weights, int64_t exchange)
{
    TORCH_CHECK(weights.is_cuda(), "All tensors must be on GPU");
    TORCH_CHECK(weights.dim() == 1 && weights.dtype() == torch::kFloat32 && weights.is_contiguous(),
                "weights must be a contiguous 1D float32 tensor");
    const c10::cuda::CUDAGuard guard(weights.device());
    auto probs = torch::empty_like(weights);
    auto total = torch::empty({1}, weights.options().dtype(torch::kFloat64));
    const int rc = puff_priorities_sm100_probs_gathered(weights.data_ptr<float>(), total.data_ptr<double>(),
                                                        probs.data_ptr<float>(), weights.size(0),
                                                        reinterpret_cast<puff_exchange*>(exchange),
                                                        at::cuda::getCurrentCUDAStream().stream());
    check_rc(rc, "puff_priority_probs_gathered");
    return {probs, total};
}

// pufferl.py:363, 373-375, 408-409 for sampled segment indices.
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor>
puff_minibatch_gather_cuda(torch::Tensor advantages, torch::Tensor values, torch::Tensor prio_probs,
                           torch::Tensor idx, double anneal_beta, int64_t prio_segments)
{
    TORCH_CHECK(advantages.is_cuda(), "All tensors must be on GPU");
    TORCH_CHECK(advantages.dim() == 2 && values.dim() == 2 && advantages.sizes() == values.sizes(),
                "advantages and values must be 2D of one shape");
    TORCH_CHECK(prio_probs.dim() == 1 && prio_probs.size(0) == advantages.size(0), "prio_probs must be [segments]");
    TORCH_CHECK(idx.dim() == 1 && idx.dtype() == torch::kInt64, "idx must be a 1D int64 tensor");
    for (const torch::Tensor& t : {advantages, values, prio_probs}) {
        TORCH_CHECK(t.dtype() == torch::kFloat32, "All tensors must be float32");
        TORCH_CHECK(t.is_contiguous(), "All tensors must be contiguous");
        TORCH_CHECK(t.device() == advantages.device(), "All tensors must be on same device");
    }
    TORCH_CHECK(idx.is_contiguous() && idx.device() == advantages.device(), "idx must be contiguous on the same device");
    const int64_t S = advantages.size(0), H = advantages.size(1), M = idx.size(0);
    int rc;
    torch::Tensor mb_values, mb_returns, mb_raw, mb_norm, mb_prio;
    {
        const c10::cuda::CUDAGuard guard(advantages.device());
        const auto opts = advantages.options();
        mb_values = torch::empty({M, H}, opts);
        mb_returns = torch::empty({M, H}, opts);
        mb_raw = torch::empty({M, H}, opts);
        mb_norm = torch::empty({M, H}, opts);
        mb_prio = torch::empty({M, 1}, opts);
        const size_t sbytes = puff_minibatch_sm100_scratch_bytes(M);
        auto scratch = torch::empty({static_cast<int64_t>((sbytes + 7) / 8)}, opts.dtype(torch::kFloat64));
        // prio_segments < 0: the probabilities were normalised over this tensor's own rows
        rc = puff_minibatch_sm100_gather_ex(advantages.data_ptr<float>(), values.data_ptr<float>(),
                                         prio_probs.data_ptr<float>(),
                                         reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()),
                                         mb_values.data_ptr<float>(), mb_returns.data_ptr<float>(),
                                         mb_raw.data_ptr<float>(), mb_norm.data_ptr<float>(), mb_prio.data_ptr<float>(),
                                         static_cast<float>(anneal_beta), S, prio_segments < 0 ? S : prio_segments, H, M,
                                         scratch.data_ptr<double>(), sbytes, at::cuda::getCurrentCUDAStream().stream());
    }
    check_rc(rc, "puff_minibatch_gather");
    return {mb_values, mb_returns, mb_raw, mb_norm, mb_prio};
}

// pufferl.py:275, 294-296 for a contiguous block of rows.
void puff_rollout_write_cuda(torch::Tensor rewards, torch::Tensor terminals, torch::Tensor values,
                             torch::Tensor step_rewards, torch::Tensor step_dones, torch::Tensor step_values,
                             int64_t row_begin, int64_t column, double reward_clip)
{
    TORCH_CHECK(rewards.is_cuda(), "All tensors must be on GPU");
    for (const torch::Tensor& t : {rewards, terminals, values}) {
        TORCH_CHECK(t.dim() == 2 && t.sizes() == rewards.sizes(), "buffers must be 2D of one shape");
        TORCH_CHECK(t.dtype() == torch::kFloat32 && t.is_contiguous(), "buffers must be contiguous float32");
        TORCH_CHECK(t.device() == rewards.device(), "All tensors must be on same device");
    }
    const int64_t n = step_rewards.numel();
    TORCH_CHECK(step_dones.numel() == n && step_values.numel() == n, "step tensors must have one entry per row");
    TORCH_CHECK(step_rewards.dtype() == torch::kFloat32 && step_values.dtype() == torch::kFloat32,
                "step rewards and values must be float32");
    TORCH_CHECK(step_dones.dtype() == torch::kBool || step_dones.dtype() == torch::kUInt8, "step dones must be bool");
    for (const torch::Tensor& t : {step_rewards, step_dones, step_values}) {
        TORCH_CHECK(t.is_contiguous() && t.device() == rewards.device(), "step tensors must be contiguous on the same device");
    }
    int rc;
    {
        const c10::cuda::CUDAGuard guard(rewards.device());
        rc = puff_rollout_sm100_write(rewards.data_ptr<float>(), terminals.data_ptr<float>(), values.data_ptr<float>(),
                                      step_rewards.data_ptr<float>(),
                                      static_cast<const unsigned char*>(step_dones.data_ptr()),
                                      step_values.data_ptr<float>(), row_begin, n, column, rewards.size(0),
                                      rewards.size(1), static_cast<float>(reward_clip),
                                      at::cuda::getCurrentCUDAStream().stream());
    }
    check_rc(rc, "puff_rollout_write");
}

// Shape-only kernels so the ops can be traced (torch.compile / fake tensors).
void compute_puff_advantage_meta(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor,
                                 double, double, double, double) {}
void compute_puff_advantage_prio_meta(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor,
                                      torch::Tensor, double, double, double, double) {}
void compute_puff_advantage_fill_meta(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor,
                                      std::optional<torch::Tensor>, double, double, double, double) {}
void puff_rollout_write_meta(torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor,
                             int64_t, int64_t, double) {}
std::tuple<torch::Tensor, torch::Tensor> puff_priority_weights_meta(torch::Tensor seg_abs_sum, double)
{
    return {torch::empty_like(seg_abs_sum), torch::empty({1}, seg_abs_sum.options().dtype(torch::kFloat64))};
}
torch::Tensor puff_priority_probs_meta(torch::Tensor weights, torch::Tensor) { return torch::empty_like(weights); }
torch::Tensor puff_priority_weights_push_meta(torch::Tensor seg_abs_sum, double, int64_t) { return torch::empty_like(seg_abs_sum); }
std::tuple<torch::Tensor, torch::Tensor> puff_priority_probs_gathered_meta(torch::Tensor weights, int64_t)
{
    return {torch::empty_like(weights), torch::empty({1}, weights.options().dtype(torch::kFloat64))};
}
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor>
puff_minibatch_gather_meta(torch::Tensor advantages, torch::Tensor, torch::Tensor, torch::Tensor idx, double, int64_t)
{
    const int64_t M = idx.size(0), H = advantages.size(1);
    const auto o = advantages.options();
    return {torch::empty({M, H}, o), torch::empty({M, H}, o), torch::empty({M, H}, o), torch::empty({M, H}, o),
            torch::empty({M, 1}, o)};
}

TORCH_LIBRARY(pufferlib, m)
{
    // byte-identical to pufferlib.cpp:88
    m.def("compute_puff_advantage(Tensor(a!) values, Tensor(b!) rewards, Tensor(c!) dones, Tensor(d!) importance, Tensor(e!) advantages, float gamma, float lambda, float rho_clip, float c_clip) -> ()");
    m.def("compute_puff_advantage_prio(Tensor values, Tensor rewards, Tensor dones, Tensor importance, Tensor(a!) advantages, Tensor(b!) seg_abs_sum, float gamma, float lambda, float rho_clip, float c_clip) -> ()");
    m.def("compute_puff_advantage_fill(Tensor values, Tensor rewards, Tensor dones, Tensor importance, Tensor(a!) advantages, Tensor(b!)? seg_abs_sum, float gamma, float lambda, float rho_clip, float c_clip) -> ()");
    m.def("puff_set_variant(int variant) -> int", &puff_set_variant);
    m.def("puff_priority_weights(Tensor seg_abs_sum, float alpha) -> (Tensor, Tensor)");
    m.def("puff_priority_probs(Tensor weights, Tensor total_w) -> Tensor");
    m.def("puff_priority_weights_push(Tensor seg_abs_sum, float alpha, int exchange) -> Tensor");
    m.def("puff_priority_probs_gathered(Tensor weights, int exchange) -> (Tensor, Tensor)");
    m.def("puff_rollout_write(Tensor(a!) rewards, Tensor(b!) terminals, Tensor(c!) values, Tensor step_rewards, Tensor step_dones, Tensor step_values, int row_begin, int column, float reward_clip) -> ()");
    m.def("puff_minibatch_gather(Tensor advantages, Tensor values, Tensor prio_probs, Tensor idx, float anneal_beta, int prio_segments=-1) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(pufferlib, CUDA, m)
{
    m.impl("compute_puff_advantage", &compute_puff_advantage_cuda);
    m.impl("compute_puff_advantage_prio", &compute_puff_advantage_prio_cuda);
    m.impl("compute_puff_advantage_fill", &compute_puff_advantage_fill_cuda);
    m.impl("puff_priority_weights", &puff_priority_weights_cuda);
    m.impl("puff_priority_probs", &puff_priority_probs_cuda);
    m.impl("puff_priority_weights_push", &puff_priority_weights_push_cuda);
    m.impl("puff_priority_probs_gathered", &puff_priority_probs_gathered_cuda);
    m.impl("puff_minibatch_gather", &puff_minibatch_gather_cuda);
    m.impl("puff_rollout_write", &puff_rollout_write_cuda);
}

TORCH_LIBRARY_IMPL(pufferlib, Meta, m)
{
    m.impl("compute_puff_advantage", &compute_puff_advantage_meta);
    m.impl("compute_puff_advantage_prio", &compute_puff_advantage_prio_meta);
    m.impl("compute_puff_advantage_fill", &compute_puff_advantage_fill_meta);
    m.impl("puff_rollout_write", &puff_rollout_write_meta);
    m.impl("puff_priority_weights", &puff_priority_weights_meta);
    m.impl("puff_priority_probs", &puff_priority_probs_meta);
    m.impl("puff_priority_weights_push", &puff_priority_weights_push_meta);
    m.impl("puff_priority_probs_gathered", &puff_priority_probs_gathered_meta);
    m.impl("puff_minibatch_gather", &puff_minibatch_gather_meta);
}

}  // namespace pufferlib_b200
