// cusync::b200::Conv2dFprop -- host handle of the library's tile-synchronised 3x3 forward convolution, with the
// call pattern of the reference's cutlass::conv::device::CuSyncImplicitGemmConvolution
// (conv/device/cusyncimplicit_gemm_convolution.h:51-319, used at ml-bench/volta_conv2d/resnet.cu:659-700):
//
//   Conv2dFprop::Arguments args{stage, problem_size, x, filter, y, y, {alpha, beta}};
//   conv.can_implement(args); conv.initialize(args, workspace);
//   conv(stream);                          // or conv.run(stream)
//   conv.params_.custage.incrementIter();
//
// CUTLASS types are replaced by small PODs; tensors are NHWC / KRSC fp16 device pointers.  The stage grid is
// conv2dGridShape(problem) and the policies take TileM = conv2dTileM(problem), TileN = conv2dTileN(problem)
// (64 for a 64-channel layer).
#pragma once

#include <cuda_runtime_api.h>
#include <stdint.h>

#include "../cusync_b200.h"
#include "cusync.h"
#include "gemm.h"

namespace cusync {
namespace b200 {

// cutlass::conv::Conv2dProblemSize as resnet.cu builds it: input {N, H, W, C}, filter {K, R, S, C}, padding,
// stride; the output has the input's H and W (stride 1, padding 1).
struct Conv2dProblemSize {
  int N, H, W, C, K, R, S, pad, stride;
  Conv2dProblemSize() : N(0), H(0), W(0), C(0), K(0), R(3), S(3), pad(1), stride(1) {}
  Conv2dProblemSize(int n, int h, int w, int c, int k, int r = 3, int s = 3, int pad_ = 1, int stride_ = 1)
      : N(n), H(h), W(w), C(c), K(k), R(r), S(s), pad(pad_), stride(stride_) {}
};

// Output pixels per M tile (whole image rows) and the stage grid (N tiles, M tiles, 1) of the implicit GEMM.
inline int conv2dTileM(const Conv2dProblemSize& p) { return cusync_conv2d_tile_rows_hw(p.H, p.W) * p.W; }
inline int conv2dTileN(const Conv2dProblemSize& p) { return cusync_conv2d_default_tile_n(p.N, p.H, p.W, p.C, p.K); }
inline dim3 conv2dGridShape(const Conv2dProblemSize& p) {
  const int rows = cusync_conv2d_tile_rows_hw(p.H, p.W);
  const int tile_n = cusync_conv2d_default_tile_n(p.N, p.H, p.W, p.C, p.K);
  return dim3(tile_n > 0 ? p.K / tile_n : 0, rows > 0 ? p.N * (p.H / rows) : 0, 1);
}

template <typename CuStageT, int EpilogueKind = EpilogueNone>
class Conv2dFprop {
 public:
  struct Arguments {
    CuStageT custage;
    Conv2dProblemSize problem_size;
    void* ref_A;   // activations x[N, H, W, C]
    void* ref_B;   // filter [K, R, S, C]
    void* ref_C;   // unused (beta = 0)
    void* ref_D;   // output y[N, H, W, K]
    EpilogueParams epilogue;
    Arguments() : ref_A(nullptr), ref_B(nullptr), ref_C(nullptr), ref_D(nullptr), epilogue{1.0f, 0.0f} {}
    Arguments(CuStageT stage, Conv2dProblemSize problem, void* x, void* filter, void* c, void* y,
              EpilogueParams epi = EpilogueParams{1.0f, 0.0f})
        : custage(stage), problem_size(problem), ref_A(x), ref_B(filter), ref_C(c), ref_D(y), epilogue(epi) {}
  };

  // Public, as in the reference: callers increment params_.custage after a run.
  struct Params { CuStageT custage; } params_;

  Conv2dFprop() : plan_(nullptr) {}

  static Status can_implement(const Arguments& a) {
    const Conv2dProblemSize& p = a.problem_size;
    if (EpilogueKind != EpilogueNone && EpilogueKind != EpilogueRelu) return Status::kErrorNotSupported;
    if (a.epilogue.alpha != 1.0f || a.epilogue.beta != 0.0f) return Status::kErrorNotSupported;
    if (p.N <= 0 || p.H <= 0 || p.W <= 0 || p.C <= 0 || p.K <= 0) return Status::kErrorInvalidProblem;
    if (p.R != 3 || p.S != 3 || p.pad != 1 || p.stride != 1 || p.C % 64 || p.K % 64) return Status::kErrorNotSupported;
    const int rows = cusync_conv2d_tile_rows_hw(p.H, p.W);
    if (rows == 0) return Status::kErrorNotSupported;
    return Status::kSuccess;
  }

  static size_t get_workspace_size(const Arguments&) { return 0; }

  Status initialize(const Arguments& a, void* workspace = nullptr, cudaStream_t stream = nullptr) {
    (void)workspace; (void)stream;
    Status s = can_implement(a);
    if (s != Status::kSuccess) return s;
    destroy();
    params_.custage = a.custage;
    const Conv2dProblemSize& p = a.problem_size;
    cusync_conv2d_desc_t d{};
    d.n = p.N; d.h = p.H; d.w = p.W; d.c = p.C; d.k = p.K;
    d.r = p.R; d.s = p.S; d.stride = p.stride; d.pad = p.pad;
    d.x = a.ref_A; d.filter = a.ref_B; d.y = a.ref_D;
    d.epilogue = EpilogueKind;
    d.stage = params_.custage.handle();
    int rc = cusync_conv2d_plan_create(&plan_, &d);
    if (rc == CUSYNC_ERROR_UNSUPPORTED) return Status::kErrorNotSupported;
    return rc == CUSYNC_SUCCESS ? Status::kSuccess : Status::kErrorInternal;
  }

  Status run(cudaStream_t stream = nullptr) {
    if (plan_ == nullptr) return Status::kErrorInternal;
    // The launch reads the run counter of the copy held in params_.
    if (params_.custage.handle()) cusync_stage_set_iter(params_.custage.handle(), params_.custage.currentIter());
    int rc = cusync_conv2d_run(plan_, reinterpret_cast<cusync_stream_t>(stream));
    return rc == CUSYNC_SUCCESS ? Status::kSuccess : Status::kErrorInternal;
  }
  Status operator()(cudaStream_t stream = nullptr) { return run(stream); }
  // The launch as a programmatic dependent of the producer kernel ahead of it in `stream` (consumers only).
  Status runDependent(cudaStream_t stream = nullptr) {
    if (plan_ == nullptr) return Status::kErrorInternal;
    if (params_.custage.handle()) cusync_stage_set_iter(params_.custage.handle(), params_.custage.currentIter());
    int rc = cusync_conv2d_run_dependent(plan_, reinterpret_cast<cusync_stream_t>(stream));
    return rc == CUSYNC_SUCCESS ? Status::kSuccess : Status::kErrorInternal;
  }

  uint32_t numCtas() const { return cusync_conv2d_plan_num_ctas(plan_); }
  void destroy() { if (plan_) { cusync_conv2d_plan_destroy(plan_); plan_ = nullptr; } }

 private:
  cusync_conv2d_plan_t* plan_;
};

}  // namespace b200
}  // namespace cusync
