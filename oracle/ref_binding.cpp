// Python binding for the parts of the reference's own CUDA sources that compile with this image's toolchain
// (cuda/src/quantization.cu, SDDMM.cu, QGEMM_backward.cu, SPMM.cu of the Tango repository).  The reference's
// binding table (cuda/src/cuda.cpp:182-204) cannot be used as it is because it also names the forward GEMM, whose
// source does not compile against current CUTLASS headers; this file declares the entry points that do exist and
// exposes them under the reference's names.  Test infrastructure: it produces the fixtures that pin the CPU oracle.
#include <cstdint>
#include <string>
#include <torch/extension.h>

// cuda/src/quantization.cu
void quantize_impl(torch::Tensor &out, torch::Tensor &in, torch::Tensor &scale);
torch::Tensor get_scale_impl(torch::Tensor &in);
torch::Tensor transpose_quant_impl(torch::Tensor &in, torch::Tensor &scale, int64_t nrow, int64_t ncol);
// cuda/src/SDDMM.cu
void mySDDMM_int8_impl(std::string &op, torch::Tensor &out, torch::Tensor &scaleOut, torch::Tensor &src,
                       torch::Tensor &dst, torch::Tensor &U, torch::Tensor &V, torch::Tensor &scaleU,
                       torch::Tensor &scaleV);
// cuda/src/QGEMM_backward.cu
void QGEMM_backward_gradX_impl(torch::Tensor &dX, torch::Tensor &dY, torch::Tensor &W, torch::Tensor &scaledY,
                               torch::Tensor &scaleW);
void QGEMM_backward_gradW_impl(torch::Tensor &dW, torch::Tensor &dY, torch::Tensor &X, torch::Tensor &scaledY,
                               torch::Tensor &scaleX);
#ifdef TANGO_REF_WITH_SPMM
// cuda/src/SPMM.cu
void cusp_SPMM_csr_impl(torch::Tensor &out, const torch::Tensor &indptr, const torch::Tensor &indices,
                        const torch::Tensor &U, const torch::Tensor &scaleU);
torch::Tensor multi_cusparse_SPMM_broadcastE_impl(const torch::Tensor &indptr, const torch::Tensor &indices,
                                                  const torch::Tensor &N, const torch::Tensor &E_T,
                                                  const torch::Tensor &scale);
void incidence_SPMM_impl(torch::Tensor &out, const torch::Tensor &src, const torch::Tensor &dst,
                         const torch::Tensor &E, const torch::Tensor &scale);
#endif

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("quantize", [](torch::Tensor out, torch::Tensor in, torch::Tensor scale) { quantize_impl(out, in, scale); });
    m.def("get_scale", [](torch::Tensor in) { return get_scale_impl(in); });
    m.def("transpose_quant", [](torch::Tensor in, torch::Tensor scale, int64_t nrow, int64_t ncol) {
        return transpose_quant_impl(in, scale, nrow, ncol);
    });
    m.def("mySDDMM_int8", [](std::string op, torch::Tensor out, torch::Tensor scaleOut, torch::Tensor src,
                             torch::Tensor dst, torch::Tensor U, torch::Tensor V, torch::Tensor scaleU,
                             torch::Tensor scaleV) {
        mySDDMM_int8_impl(op, out, scaleOut, src, dst, U, V, scaleU, scaleV);
    });
    m.def("QGEMM_backward_gradX", [](torch::Tensor dX, torch::Tensor dY, torch::Tensor W, torch::Tensor sdY,
                                     torch::Tensor sW) { QGEMM_backward_gradX_impl(dX, dY, W, sdY, sW); });
    m.def("QGEMM_backward_gradW", [](torch::Tensor dW, torch::Tensor dY, torch::Tensor X, torch::Tensor sdY,
                                     torch::Tensor sX) { QGEMM_backward_gradW_impl(dW, dY, X, sdY, sX); });
#ifdef TANGO_REF_WITH_SPMM
    m.def("csr_SPMM", [](torch::Tensor out, torch::Tensor indptr, torch::Tensor indices, torch::Tensor U,
                         torch::Tensor scaleU) { cusp_SPMM_csr_impl(out, indptr, indices, U, scaleU); });
    m.def("multi_cusparse_SPMM", [](torch::Tensor indptr, torch::Tensor indices, torch::Tensor N, torch::Tensor E_T,
                                    torch::Tensor scale) {
        return multi_cusparse_SPMM_broadcastE_impl(indptr, indices, N, E_T, scale);
    });
    m.def("incidence_SPMM", [](torch::Tensor out, torch::Tensor src, torch::Tensor dst, torch::Tensor E,
                               torch::Tensor scale) { incidence_SPMM_impl(out, src, dst, E, scale); });
    m.attr("has_spmm") = true;
#else
    m.attr("has_spmm") = false;
#endif
}
