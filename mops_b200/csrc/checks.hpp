// Host-side shape rules of the five operations, with the reference's error texts.
//
// Message formats: mops/src/internal/checks/utils.hpp:31-37 (size mismatch). The rules
// per op: checks/hpe.hpp:16-17, checks/sap.hpp:19-23, checks/opsa.hpp:17-20,
// checks/opsaw.hpp:18-24, checks/sasaw.hpp:22-29, and the *_vjp variants in the same files
// (a gradient output is checked against its primal only when it is requested).
// The reference skips the host scan of index values for "cuda_" operations because the
// arrays live on the device; here the kernels check them and report through the status
// block instead (runtime.hpp).
#ifndef MOPS_B200_CHECKS_HPP
#define MOPS_B200_CHECKS_HPP

#include <stdexcept>
#include <string>

#include "mops.hpp"

namespace mops_b200 {

template <typename TA, size_t NA, typename TB, size_t NB>
void same_size(const mops::Tensor<TA, NA>& a, const char* name_a, size_t dim_a,
               const mops::Tensor<TB, NB>& b, const char* name_b, size_t dim_b,
               const std::string& operation) {
    if (a.shape[dim_a] != b.shape[dim_b]) {
        throw std::runtime_error(
            std::string("Dimension mismatch: the sizes of ") + name_a + " along dimension " +
            std::to_string(dim_a) + " and " + name_b + " along dimension " +
            std::to_string(dim_b) + " must match in " + operation);
    }
}

// A requested gradient must have the shape of its primal.
template <typename T, size_t N>
void grad_like(const mops::Tensor<T, N>& grad, const char* grad_name,
               const mops::Tensor<T, N>& primal, const char* primal_name,
               const std::string& operation) {
    if (grad.data == nullptr) return;
    for (size_t d = 0; d < N; d++) same_size(grad, grad_name, d, primal, primal_name, d, operation);
}

inline void fits_int32(size_t value, const char* what, const std::string& operation) {
    if (value > static_cast<size_t>(INT32_MAX)) {
        throw std::runtime_error(std::string(what) + " is too large for 32-bit indices in " +
                                 operation);
    }
}

} // namespace mops_b200

#endif
