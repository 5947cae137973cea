// torch operators `torch.ops.mops.*` backed by the sm_100a kernels.
//
// Same operator namespace and schemas as the reference's mops-torch
// (mops-torch/src/register.cpp:5-38), registered the same way (a plain function that applies
// a torch::autograd::Function), so eager code, TorchScript and saved modules written against
// the reference run unchanged. Differences: all five operations have a CUDA implementation
// here (the reference has none for OPSAW and SASAW, mops-torch/src/opsaw.cpp:36-60,
// sasaw.cpp:65-97); inputs are made contiguous; kernels run on torch's current stream of the
// tensors' device without synchronising it; CPU tensors are rejected, because this build has
// no CPU implementation.
//
// Checks and error types follow mops-torch/src/utils.cpp:7-66 (same device, f32/f64 only and
// all equal, int32 indices, number of dimensions) and the per-op rules: gradients with respect
// to C are refused (mops-torch/src/hpe.cpp:85-91, sap.cpp:135-141, sasaw.cpp:158-164); second
// derivatives exist for HPE, SAP and OPSA (the operations whose _vjp_vjp the reference declares);
// OPSAW and SASAW refuse them, as the reference does.
#include <string>
#include <vector>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/script.h>

#include "../../include/mops.h"
#include "mops.hpp"

namespace {

using torch::Tensor;
using torch::autograd::AutogradContext;
using tensor_list = std::vector<Tensor>;

void same_device(const tensor_list& tensors) {
    for (const auto& t : tensors) {
        if (t.device() != tensors[0].device()) {
            C10_THROW_ERROR(ValueError, "All tensors must be on the same device, found " +
                                            t.device().str() + " and " + tensors[0].device().str());
        }
    }
}

void floating(const tensor_list& tensors) {
    const auto dtype = tensors[0].dtype();
    if (dtype != torch::kF64 && dtype != torch::kF32) {
        C10_THROW_ERROR(TypeError, "Found dtype " + std::string(dtype.name()) +
                                       ", only float32 and float64 are supported");
    }
    for (const auto& t : tensors) {
        if (t.dtype() != dtype) {
            C10_THROW_ERROR(TypeError,
                            "All floating point tensors must be of the same dtype, found " +
                                std::string(t.dtype().name()) + " and " + std::string(dtype.name()));
        }
    }
}

void int32_indices(const tensor_list& tensors) {
    for (const auto& t : tensors) {
        if (t.dtype() != torch::kI32) {
            C10_THROW_ERROR(TypeError, "All index tensors must be of type int32, found " +
                                           std::string(t.dtype().name()));
        }
    }
}

void ndim(const Tensor& t, int64_t expected, const char* name, const char* op) {
    if (t.dim() != expected) {
        C10_THROW_ERROR(ValueError, std::string("Expected ") + name + " to have " +
                                        std::to_string(expected) + " dimensions, in " + op +
                                        ", found " + std::to_string(t.dim()));
    }
}

void cuda_only(const Tensor& t, const char* op) {
    if (!t.device().is_cuda()) {
        C10_THROW_ERROR(ValueError, std::string(op) + " is not implemented for device " +
                                        t.device().str() +
                                        ": this build of mops provides the CUDA (sm_100a) "
                                        "implementations only");
    }
}

template <typename T, size_t N> mops::Tensor<T, N> view(const Tensor& t) {
    mops::Tensor<T, N> out;
    out.data = t.defined() ? t.data_ptr<T>() : nullptr;
    for (size_t d = 0; d < N; d++) out.shape[d] = t.defined() ? static_cast<size_t>(t.size(d)) : 0;
    return out;
}

// Runs `body` with the device of `like` current and the library pointed at torch's current
// stream, without waiting for the kernels.
template <typename F> void on_stream_of(const Tensor& like, F&& body) {
    const c10::cuda::CUDAGuard guard(like.device());
    void* previous_stream = mops_b200_get_stream();
    const int previous_wait = mops_b200_get_wait();
    mops_b200_set_stream(at::cuda::getCurrentCUDAStream().stream());
    mops_b200_set_wait(0);
    try {
        body();
    } catch (...) {
        mops_b200_set_stream(previous_stream);
        mops_b200_set_wait(previous_wait);
        throw;
    }
    mops_b200_set_stream(previous_stream);
    mops_b200_set_wait(previous_wait);
}

Tensor maybe_empty_like(const Tensor& t) { return t.requires_grad() ? torch::empty_like(t) : Tensor(); }

// Outputs of an autograd Function must be defined tensors: a gradient that was not requested
// is returned as an empty placeholder and turned back into "no gradient" by the caller.
Tensor defined(const Tensor& t, const Tensor& like) {
    return t.defined() ? t : torch::empty({0}, like.options());
}
Tensor requested(const Tensor& t) { return t.defined() && t.numel() == 0 ? Tensor() : t; }

[[noreturn]] void no_second_derivative(const char* op) {
    C10_THROW_ERROR(NotImplementedError,
                    std::string("second derivatives are not supported in CUDA for ") + op);
}

// =============================================================================== HPE
struct HpeBackward : torch::autograd::Function<HpeBackward> {
    static tensor_list forward(AutogradContext* ctx, Tensor grad_output, Tensor A, Tensor C,
                               Tensor indices_A) {
        if (C.requires_grad()) {
            C10_THROW_ERROR(ValueError, "gradients with respect to the coefficients C are not "
                                        "supported in homogeneous_polynomial_evaluation");
        }
        Tensor grad_A = maybe_empty_like(A);
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), "homogeneous_polynomial_evaluation_vjp", [&] {
                mops::cuda::homogeneous_polynomial_evaluation_vjp<scalar_t>(
                    view<scalar_t, 2>(grad_A), view<scalar_t, 1>(grad_output), view<scalar_t, 2>(A),
                    view<scalar_t, 1>(C), view<int32_t, 2>(indices_A));
            });
        });
        if (grad_output.requires_grad() || A.requires_grad()) {
            ctx->save_for_backward({grad_output, A, C, indices_A});
        }
        return {defined(grad_A, A)};
    }
    static tensor_list backward(AutogradContext* ctx, tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        Tensor grad_output = saved[0], A = saved[1], C = saved[2], indices_A = saved[3];
        // a placeholder output (gradient not requested in the first backward) has no gradient
        Tensor gg_A = grads[0].defined() && grads[0].sizes() == A.sizes() ? grads[0].contiguous()
                                                                           : Tensor();
        Tensor gg_output = maybe_empty_like(grad_output), grad_A_2 = maybe_empty_like(A);
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), "homogeneous_polynomial_evaluation_vjp_vjp", [&] {
                mops::cuda::homogeneous_polynomial_evaluation_vjp_vjp<scalar_t>(
                    view<scalar_t, 1>(gg_output), view<scalar_t, 2>(grad_A_2),
                    view<scalar_t, 2>(gg_A), view<scalar_t, 1>(grad_output), view<scalar_t, 2>(A),
                    view<scalar_t, 1>(C), view<int32_t, 2>(indices_A));
            });
        });
        return {gg_output, grad_A_2, Tensor(), Tensor()};
    }
};

struct Hpe : torch::autograd::Function<Hpe> {
    static Tensor forward(AutogradContext* ctx, Tensor A, Tensor C, Tensor indices_A) {
        static constexpr const char* op = "homogeneous_polynomial_evaluation";
        same_device({A, C, indices_A});
        floating({A, C});
        int32_indices({indices_A});
        ndim(A, 2, "A", op);
        ndim(C, 1, "C", op);
        ndim(indices_A, 2, "indices_A", op);
        cuda_only(A, op);
        A = A.contiguous();
        C = C.contiguous();
        indices_A = indices_A.contiguous();
        Tensor output = torch::empty({A.size(0)}, A.options());
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), op, [&] {
                mops::cuda::homogeneous_polynomial_evaluation<scalar_t>(
                    view<scalar_t, 1>(output), view<scalar_t, 2>(A), view<scalar_t, 1>(C),
                    view<int32_t, 2>(indices_A));
            });
        });
        if (A.requires_grad() || C.requires_grad()) ctx->save_for_backward({A, C, indices_A});
        return output;
    }
    static tensor_list backward(AutogradContext* ctx, tensor_list grad_outputs) {
        auto saved = ctx->get_saved_variables();
        auto results = HpeBackward::apply(grad_outputs[0].contiguous(), saved[0], saved[1], saved[2]);
        return {requested(results[0]), Tensor(), Tensor()};
    }
};

// =============================================================================== SAP
struct SapBackward : torch::autograd::Function<SapBackward> {
    static tensor_list forward(AutogradContext* ctx, Tensor grad_output, Tensor A, Tensor B,
                               Tensor C, Tensor indices_A, Tensor indices_B,
                               Tensor indices_output) {
        if (C.requires_grad()) {
            C10_THROW_ERROR(ValueError, "gradients with respect to the coefficients C are not "
                                        "supported in sparse_accumulation_of_products");
        }
        Tensor grad_A = maybe_empty_like(A), grad_B = maybe_empty_like(B);
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), "sparse_accumulation_of_products_vjp", [&] {
                mops::cuda::sparse_accumulation_of_products_vjp<scalar_t>(
                    view<scalar_t, 2>(grad_A), view<scalar_t, 2>(grad_B),
                    view<scalar_t, 2>(grad_output), view<scalar_t, 2>(A), view<scalar_t, 2>(B),
                    view<scalar_t, 1>(C), view<int32_t, 1>(indices_A), view<int32_t, 1>(indices_B),
                    view<int32_t, 1>(indices_output));
            });
        });
        if (grad_output.requires_grad() || A.requires_grad() || B.requires_grad()) {
            ctx->save_for_backward({grad_output, A, B, C, indices_A, indices_B, indices_output});
        }
        return {defined(grad_A, A), defined(grad_B, A)};
    }
    static tensor_list backward(AutogradContext* ctx, tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        Tensor grad_output = saved[0], A = saved[1], B = saved[2], C = saved[3];
        Tensor indices_A = saved[4], indices_B = saved[5], indices_output = saved[6];
        // a placeholder output (gradient not requested in the first backward) has no gradient
        Tensor gg_A = grads[0].defined() && grads[0].sizes() == A.sizes() ? grads[0].contiguous()
                                                                           : Tensor();
        Tensor gg_B = grads[1].defined() && grads[1].sizes() == B.sizes() ? grads[1].contiguous()
                                                                           : Tensor();
        Tensor gg_output = maybe_empty_like(grad_output);
        Tensor grad_A_2 = maybe_empty_like(A), grad_B_2 = maybe_empty_like(B);
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), "sparse_accumulation_of_products_vjp_vjp", [&] {
                mops::cuda::sparse_accumulation_of_products_vjp_vjp<scalar_t>(
                    view<scalar_t, 2>(gg_output), view<scalar_t, 2>(grad_A_2),
                    view<scalar_t, 2>(grad_B_2), view<scalar_t, 2>(gg_A), view<scalar_t, 2>(gg_B),
                    view<scalar_t, 2>(grad_output), view<scalar_t, 2>(A), view<scalar_t, 2>(B),
                    view<scalar_t, 1>(C), view<int32_t, 1>(indices_A), view<int32_t, 1>(indices_B),
                    view<int32_t, 1>(indices_output));
            });
        });
        return {gg_output, grad_A_2, grad_B_2, Tensor(), Tensor(), Tensor(), Tensor()};
    }
};

struct Sap : torch::autograd::Function<Sap> {
    static Tensor forward(AutogradContext* ctx, Tensor A, Tensor B, Tensor C, Tensor indices_A,
                          Tensor indices_B, Tensor indices_output, int64_t output_size) {
        static constexpr const char* op = "sparse_accumulation_of_products";
        same_device({A, B, C, indices_A, indices_B, indices_output});
        floating({A, B, C});
        int32_indices({indices_A, indices_B, indices_output});
        ndim(A, 2, "A", op);
        ndim(B, 2, "B", op);
        ndim(C, 1, "C", op);
        ndim(indices_A, 1, "indices_A", op);
        ndim(indices_B, 1, "indices_B", op);
        ndim(indices_output, 1, "indices_output", op);
        cuda_only(A, op);
        A = A.contiguous();
        B = B.contiguous();
        C = C.contiguous();
        indices_A = indices_A.contiguous();
        indices_B = indices_B.contiguous();
        indices_output = indices_output.contiguous();
        Tensor output = torch::empty({A.size(0), output_size}, A.options());
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), op, [&] {
                mops::cuda::sparse_accumulation_of_products<scalar_t>(
                    view<scalar_t, 2>(output), view<scalar_t, 2>(A), view<scalar_t, 2>(B),
                    view<scalar_t, 1>(C), view<int32_t, 1>(indices_A), view<int32_t, 1>(indices_B),
                    view<int32_t, 1>(indices_output));
            });
        });
        if (A.requires_grad() || B.requires_grad() || C.requires_grad()) {
            ctx->save_for_backward({A, B, C, indices_A, indices_B, indices_output});
        }
        return output;
    }
    static tensor_list backward(AutogradContext* ctx, tensor_list grad_outputs) {
        auto s = ctx->get_saved_variables();
        auto r = SapBackward::apply(grad_outputs[0].contiguous(), s[0], s[1], s[2], s[3], s[4], s[5]);
        return {requested(r[0]), requested(r[1]), Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
    }
};

// =============================================================================== OPSA
struct OpsaBackward : torch::autograd::Function<OpsaBackward> {
    static tensor_list forward(AutogradContext* ctx, Tensor grad_output, Tensor A, Tensor B,
                               Tensor indices_output) {
        Tensor grad_A = maybe_empty_like(A), grad_B = maybe_empty_like(B);
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), "outer_product_scatter_add_vjp", [&] {
                mops::cuda::outer_product_scatter_add_vjp<scalar_t>(
                    view<scalar_t, 2>(grad_A), view<scalar_t, 2>(grad_B),
                    view<scalar_t, 3>(grad_output), view<scalar_t, 2>(A), view<scalar_t, 2>(B),
                    view<int32_t, 1>(indices_output));
            });
        });
        if (grad_output.requires_grad() || A.requires_grad() || B.requires_grad()) {
            ctx->save_for_backward({grad_output, A, B, indices_output});
        }
        return {defined(grad_A, A), defined(grad_B, A)};
    }
    static tensor_list backward(AutogradContext* ctx, tensor_list grads) {
        auto saved = ctx->get_saved_variables();
        Tensor grad_output = saved[0], A = saved[1], B = saved[2], indices_output = saved[3];
        // a placeholder output (gradient not requested in the first backward) has no gradient
        Tensor gg_A = grads[0].defined() && grads[0].sizes() == A.sizes() ? grads[0].contiguous()
                                                                           : Tensor();
        Tensor gg_B = grads[1].defined() && grads[1].sizes() == B.sizes() ? grads[1].contiguous()
                                                                           : Tensor();
        Tensor gg_output = maybe_empty_like(grad_output);
        Tensor grad_A_2 = maybe_empty_like(A), grad_B_2 = maybe_empty_like(B);
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), "outer_product_scatter_add_vjp_vjp", [&] {
                mops::cuda::outer_product_scatter_add_vjp_vjp<scalar_t>(
                    view<scalar_t, 3>(gg_output), view<scalar_t, 2>(grad_A_2),
                    view<scalar_t, 2>(grad_B_2), view<scalar_t, 2>(gg_A), view<scalar_t, 2>(gg_B),
                    view<scalar_t, 3>(grad_output), view<scalar_t, 2>(A), view<scalar_t, 2>(B),
                    view<int32_t, 1>(indices_output));
            });
        });
        return {gg_output, grad_A_2, grad_B_2, Tensor()};
    }
};

struct Opsa : torch::autograd::Function<Opsa> {
    static Tensor forward(AutogradContext* ctx, Tensor A, Tensor B, Tensor indices_output,
                          int64_t output_size) {
        static constexpr const char* op = "outer_product_scatter_add";
        same_device({A, B, indices_output});
        floating({A, B});
        int32_indices({indices_output});
        ndim(A, 2, "A", op);
        ndim(B, 2, "B", op);
        ndim(indices_output, 1, "indices_output", op);
        cuda_only(A, op);
        A = A.contiguous();
        B = B.contiguous();
        indices_output = indices_output.contiguous();
        Tensor output = torch::empty({output_size, A.size(1), B.size(1)}, A.options());
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), op, [&] {
                mops::cuda::outer_product_scatter_add<scalar_t>(
                    view<scalar_t, 3>(output), view<scalar_t, 2>(A), view<scalar_t, 2>(B),
                    view<int32_t, 1>(indices_output));
            });
        });
        if (A.requires_grad() || B.requires_grad()) ctx->save_for_backward({A, B, indices_output});
        return output;
    }
    static tensor_list backward(AutogradContext* ctx, tensor_list grad_outputs) {
        auto s = ctx->get_saved_variables();
        auto r = OpsaBackward::apply(grad_outputs[0].contiguous(), s[0], s[1], s[2]);
        return {requested(r[0]), requested(r[1]), Tensor(), Tensor()};
    }
};

// =============================================================================== OPSAW
struct OpsawBackward : torch::autograd::Function<OpsawBackward> {
    static tensor_list forward(AutogradContext*, Tensor grad_output, Tensor A, Tensor B, Tensor W,
                               Tensor indices_W, Tensor indices_output) {
        Tensor grad_A = maybe_empty_like(A), grad_B = maybe_empty_like(B),
               grad_W = maybe_empty_like(W);
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), "outer_product_scatter_add_with_weights_vjp", [&] {
                mops::cuda::outer_product_scatter_add_with_weights_vjp<scalar_t>(
                    view<scalar_t, 2>(grad_A), view<scalar_t, 2>(grad_B), view<scalar_t, 2>(grad_W),
                    view<scalar_t, 3>(grad_output), view<scalar_t, 2>(A), view<scalar_t, 2>(B),
                    view<scalar_t, 2>(W), view<int32_t, 1>(indices_W),
                    view<int32_t, 1>(indices_output));
            });
        });
        return {defined(grad_A, A), defined(grad_B, A), defined(grad_W, A)};
    }
    static tensor_list backward(AutogradContext*, tensor_list) {
        no_second_derivative("outer_product_scatter_add_with_weights");
    }
};

struct Opsaw : torch::autograd::Function<Opsaw> {
    static Tensor forward(AutogradContext* ctx, Tensor A, Tensor B, Tensor W, Tensor indices_W,
                          Tensor indices_output) {
        static constexpr const char* op = "outer_product_scatter_add_with_weights";
        same_device({A, B, W, indices_W, indices_output});
        floating({A, B, W});
        int32_indices({indices_W, indices_output});
        ndim(A, 2, "A", op);
        ndim(B, 2, "B", op);
        ndim(W, 2, "W", op);
        ndim(indices_W, 1, "indices_W", op);
        ndim(indices_output, 1, "indices_output", op);
        cuda_only(A, op);
        A = A.contiguous();
        B = B.contiguous();
        W = W.contiguous();
        indices_W = indices_W.contiguous();
        indices_output = indices_output.contiguous();
        Tensor output = torch::empty({W.size(0), A.size(1), B.size(1)}, A.options());
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), op, [&] {
                mops::cuda::outer_product_scatter_add_with_weights<scalar_t>(
                    view<scalar_t, 3>(output), view<scalar_t, 2>(A), view<scalar_t, 2>(B),
                    view<scalar_t, 2>(W), view<int32_t, 1>(indices_W),
                    view<int32_t, 1>(indices_output));
            });
        });
        if (A.requires_grad() || B.requires_grad() || W.requires_grad()) {
            ctx->save_for_backward({A, B, W, indices_W, indices_output});
        }
        return output;
    }
    static tensor_list backward(AutogradContext* ctx, tensor_list grad_outputs) {
        auto s = ctx->get_saved_variables();
        auto r = OpsawBackward::apply(grad_outputs[0].contiguous(), s[0], s[1], s[2], s[3], s[4]);
        return {requested(r[0]), requested(r[1]), requested(r[2]), Tensor(), Tensor()};
    }
};

// =============================================================================== SASAW
struct SasawBackward : torch::autograd::Function<SasawBackward> {
    static tensor_list forward(AutogradContext*, Tensor grad_output, Tensor A, Tensor B, Tensor C,
                               Tensor W, Tensor indices_A, Tensor indices_W_1, Tensor indices_W_2,
                               Tensor indices_output_1, Tensor indices_output_2) {
        if (C.requires_grad()) {
            C10_THROW_ERROR(ValueError,
                            "gradients with respect to the coefficients C are not supported in "
                            "sparse_accumulation_scatter_add_with_weights");
        }
        Tensor grad_A = maybe_empty_like(A), grad_B = maybe_empty_like(B),
               grad_W = maybe_empty_like(W);
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(
                A.scalar_type(), "sparse_accumulation_scatter_add_with_weights_vjp", [&] {
                    mops::cuda::sparse_accumulation_scatter_add_with_weights_vjp<scalar_t>(
                        view<scalar_t, 2>(grad_A), view<scalar_t, 2>(grad_B),
                        view<scalar_t, 3>(grad_W), view<scalar_t, 3>(grad_output),
                        view<scalar_t, 2>(A), view<scalar_t, 2>(B), view<scalar_t, 1>(C),
                        view<scalar_t, 3>(W), view<int32_t, 1>(indices_A),
                        view<int32_t, 1>(indices_W_1), view<int32_t, 1>(indices_W_2),
                        view<int32_t, 1>(indices_output_1), view<int32_t, 1>(indices_output_2));
                });
        });
        return {defined(grad_A, A), defined(grad_B, A), defined(grad_W, A)};
    }
    static tensor_list backward(AutogradContext*, tensor_list) {
        no_second_derivative("sparse_accumulation_scatter_add_with_weights");
    }
};

struct Sasaw : torch::autograd::Function<Sasaw> {
    static Tensor forward(AutogradContext* ctx, Tensor A, Tensor B, Tensor C, Tensor W,
                          Tensor indices_A, Tensor indices_W_1, Tensor indices_W_2,
                          Tensor indices_output_1, Tensor indices_output_2, int64_t output_size) {
        static constexpr const char* op = "sparse_accumulation_scatter_add_with_weights";
        same_device({A, B, C, W, indices_A, indices_W_1, indices_W_2, indices_output_1,
                     indices_output_2});
        floating({A, B, C, W});
        int32_indices({indices_A, indices_W_1, indices_W_2, indices_output_1, indices_output_2});
        ndim(A, 2, "A", op);
        ndim(B, 2, "B", op);
        ndim(C, 1, "C", op);
        ndim(W, 3, "W", op);
        ndim(indices_A, 1, "indices_A", op);
        ndim(indices_W_1, 1, "indices_W_1", op);
        ndim(indices_W_2, 1, "indices_W_2", op);
        ndim(indices_output_1, 1, "indices_output_1", op);
        ndim(indices_output_2, 1, "indices_output_2", op);
        cuda_only(A, op);
        A = A.contiguous();
        B = B.contiguous();
        C = C.contiguous();
        W = W.contiguous();
        indices_A = indices_A.contiguous();
        indices_W_1 = indices_W_1.contiguous();
        indices_W_2 = indices_W_2.contiguous();
        indices_output_1 = indices_output_1.contiguous();
        indices_output_2 = indices_output_2.contiguous();
        Tensor output = torch::empty({W.size(0), output_size, B.size(1)}, A.options());
        on_stream_of(A, [&] {
            AT_DISPATCH_FLOATING_TYPES(A.scalar_type(), op, [&] {
                mops::cuda::sparse_accumulation_scatter_add_with_weights<scalar_t>(
                    view<scalar_t, 3>(output), view<scalar_t, 2>(A), view<scalar_t, 2>(B),
                    view<scalar_t, 1>(C), view<scalar_t, 3>(W), view<int32_t, 1>(indices_A),
                    view<int32_t, 1>(indices_W_1), view<int32_t, 1>(indices_W_2),
                    view<int32_t, 1>(indices_output_1), view<int32_t, 1>(indices_output_2));
            });
        });
        if (A.requires_grad() || B.requires_grad() || C.requires_grad() || W.requires_grad()) {
            ctx->save_for_backward({A, B, C, W, indices_A, indices_W_1, indices_W_2,
                                    indices_output_1, indices_output_2});
        }
        return output;
    }
    static tensor_list backward(AutogradContext* ctx, tensor_list grad_outputs) {
        auto s = ctx->get_saved_variables();
        auto r = SasawBackward::apply(grad_outputs[0].contiguous(), s[0], s[1], s[2], s[3], s[4],
                                      s[5], s[6], s[7], s[8]);
        return {requested(r[0]), requested(r[1]), Tensor(), requested(r[2]), Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
    }
};

// ------------------------------------------------------------------ registered entry points
Tensor hpe(Tensor A, Tensor C, Tensor indices_A) { return Hpe::apply(A, C, indices_A); }

Tensor opsa(Tensor A, Tensor B, Tensor indices_output, int64_t output_size) {
    return Opsa::apply(A, B, indices_output, output_size);
}

Tensor sap(Tensor A, Tensor B, Tensor C, Tensor indices_A, Tensor indices_B, Tensor indices_output,
           int64_t output_size) {
    return Sap::apply(A, B, C, indices_A, indices_B, indices_output, output_size);
}

Tensor opsaw(Tensor A, Tensor B, Tensor W, Tensor indices_W, Tensor indices_output) {
    return Opsaw::apply(A, B, W, indices_W, indices_output);
}

Tensor sasaw(Tensor A, Tensor B, Tensor C, Tensor W, Tensor indices_A, Tensor indices_W_1,
             Tensor indices_W_2, Tensor indices_output_1, Tensor indices_output_2,
             int64_t output_size) {
    return Sasaw::apply(A, B, C, W, indices_A, indices_W_1, indices_W_2, indices_output_1,
                        indices_output_2, output_size);
}

} // namespace

TORCH_LIBRARY(mops, m) {
    m.def("homogeneous_polynomial_evaluation(Tensor A, Tensor C, Tensor indices_A) -> Tensor", hpe);
    m.def("outer_product_scatter_add(Tensor A, Tensor B, Tensor indices_output, int output_size) "
          "-> Tensor",
          opsa);
    m.def("sparse_accumulation_of_products(Tensor A, Tensor B, Tensor C, Tensor indices_A, "
          "Tensor indices_B, Tensor indices_output, int output_size) -> Tensor",
          sap);
    m.def("outer_product_scatter_add_with_weights(Tensor A, Tensor B, Tensor W, Tensor indices_W, "
          "Tensor indices_output) -> Tensor",
          opsaw);
    m.def("sparse_accumulation_scatter_add_with_weights(Tensor A, Tensor B, Tensor C, Tensor W, "
          "Tensor indices_A, Tensor indices_W_1, Tensor indices_W_2, Tensor indices_output_1, "
          "Tensor indices_output_2, int output_size) -> Tensor",
          sasaw);
}
