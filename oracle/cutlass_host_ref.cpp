// TEST INFRASTRUCTURE ONLY.  C entry points around NVIDIA CUTLASS's host reference kernels, so that the
// CPU oracle's arithmetic (orc_gemm_f16, orc_conv2d_3x3_nhwc_f16 in cusync_oracle.c) can be pinned to the code
// the reference itself checks its kernels against:
//   * cutlass::reference::host::Conv2dFprop with the element types of
//     src/ml-bench/volta_conv2d/resnet.cu:72-80 as called at resnet.cu:706-720
//     (half inputs, float accumulator, half epilogue compute, alpha = 1, beta = 0);
//   * cutlass::reference::host::Gemm<half, RowMajor, half, RowMajor, half, RowMajor, float, float>, the host
//     GEMM of the CUTLASS the reference builds against (its drivers' referenceMLP,
//     src/ml-bench/transformer/mlp.cu:333-379, uses the same arithmetic: fp32 accumulation in k order, one
//     rounding to half per stored element).
//   * the activation functors of cutlass/epilogue/thread/activation.h in float: GELU (the erf form that
//     LinearCombinationGELU applies, mlp.cu:140-163), SiLu and ReLu.
// CUTLASS is a third-party dependency that is NOT part of the reference tree (an empty, un-pinned submodule
// there); this file only includes its headers from wherever the build finds them (see oracle/Makefile,
// CUTLASS_ROOT) and nothing of it is copied here.  Output goes to oracle/_ref/.
#include <cstdint>

#include "cutlass/cutlass.h"
#include "cutlass/conv/conv2d_problem_size.h"
#include "cutlass/epilogue/thread/activation.h"
#include "cutlass/gemm/gemm.h"
#include "cutlass/layout/matrix.h"
#include "cutlass/layout/tensor.h"
#include "cutlass/numeric_types.h"
#include "cutlass/tensor_ref.h"
#include "cutlass/util/reference/host/convolution.h"
#include "cutlass/util/reference/host/gemm.h"

using half_t = cutlass::half_t;

extern "C" {

// C[m,n] = A[m,k] * B[k,n], all row-major half, float accumulate, alpha = 1, beta = 0.
void cutlass_ref_gemm_f16(int m, int n, int k, const void* a, int lda, const void* b, int ldb, void* c, int ldc) {
  using RowMajor = cutlass::layout::RowMajor;
  cutlass::TensorRef<half_t, RowMajor> ra(const_cast<half_t*>(static_cast<const half_t*>(a)), RowMajor(lda));
  cutlass::TensorRef<half_t, RowMajor> rb(const_cast<half_t*>(static_cast<const half_t*>(b)), RowMajor(ldb));
  cutlass::TensorRef<half_t, RowMajor> rc(static_cast<half_t*>(c), RowMajor(ldc));
  cutlass::reference::host::Gemm<half_t, RowMajor, half_t, RowMajor, half_t, RowMajor, float, float> gemm;
  gemm(cutlass::gemm::GemmCoord(m, n, k), 1.0f, ra, rb, 0.0f, rc, rc, 0.0f);
}

// y[n,h,w,k] = conv(x[n,h,w,c], filter[k,r,s,c]), NHWC / KRSC half, stride 1; the template arguments and
// alpha/beta are those of resnet.cu:706-720.
void cutlass_ref_conv2d_fprop_f16(int n, int h, int w, int c, int k, int r, int s, int pad, const void* x,
                                  const void* filter, void* y) {
  using NHWC = cutlass::layout::TensorNHWC;
  const int p = h + 2 * pad - r + 1, q = w + 2 * pad - s + 1;
  cutlass::conv::Conv2dProblemSize problem({n, h, w, c}, {k, r, s, c}, {pad, pad, pad, pad}, {1, 1}, {1, 1},
                                           {n, p, q, k}, cutlass::conv::Mode::kCrossCorrelation, 1);
  cutlass::TensorRef<half_t, NHWC> rx(const_cast<half_t*>(static_cast<const half_t*>(x)), NHWC::packed({n, h, w, c}));
  cutlass::TensorRef<half_t, NHWC> rw(const_cast<half_t*>(static_cast<const half_t*>(filter)),
                                      NHWC::packed({k, r, s, c}));
  cutlass::TensorRef<half_t, NHWC> ry(static_cast<half_t*>(y), NHWC::packed({n, p, q, k}));
  using Convert = cutlass::NumericConverter<half_t, half_t>;
  cutlass::reference::host::Conv2dFprop<half_t, NHWC, half_t, NHWC, half_t, NHWC, half_t, float, half_t, Convert>(
      problem, rx, rw, ry, ry, half_t(1.0f), half_t(0.0f));
}

// out[i] = act(in[i]) in float: kind 1 = GELU (erf), 2 = ReLu, 3 = SiLu.
void cutlass_ref_activation_f32(int kind, long long count, const float* in, float* out) {
  cutlass::epilogue::thread::GELU<float> gelu;
  cutlass::epilogue::thread::ReLu<float> relu;
  cutlass::epilogue::thread::SiLu<float> silu;
  for (long long i = 0; i < count; i++)
    out[i] = kind == 1 ? gelu(in[i]) : kind == 2 ? relu(in[i]) : kind == 3 ? silu(in[i]) : in[i];
}

}  // extern "C"
