// cusync::b200::Gemm -- host handle of the library's tile-synchronised GEMM,
// with the call pattern of the reference's cutlass::gemm::device::CuSyncGemm
// (gemm/device/cusyncgemm.h:234-599, used at ml-bench/transformer/mlp.cu:653-712):
//
//   Gemm::Arguments args{stage, {M, N, K}, refA, refB, refC, refD, {alpha, beta}, split_k};
//   gemm.can_implement(args); gemm.initialize(args, workspace);
//   gemm.run(true, NULL, stream);
//   gemm.params_.custage.incrementIter();
//
// CUTLASS types are replaced by the small PODs below; the kernels are the
// library's pre-compiled sm_100a ones, so the stage's policies must be
// built-in policies (or provide desc()).
#pragma once

#include <cuda_runtime_api.h>
#include <stdint.h>

#include "../cusync_b200.h"
#include "cusync.h"

namespace cusync {
namespace b200 {

enum class Status { kSuccess = 0, kErrorInvalidProblem, kErrorNotSupported, kErrorMisalignedOperand, kErrorInternal };

struct GemmCoord {
  int m_, n_, k_;
  GemmCoord() : m_(0), n_(0), k_(0) {}
  GemmCoord(int m, int n, int k) : m_(m), n_(n), k_(k) {}
  int m() const { return m_; }
  int n() const { return n_; }
  int k() const { return k_; }
};

// Row-major fp16 matrix: pointer + leading dimension in elements.
struct TensorRef {
  void* ptr;
  int64_t ld;
  TensorRef() : ptr(nullptr), ld(0) {}
  TensorRef(void* p, int64_t l) : ptr(p), ld(l) {}
};

struct EpilogueParams { float alpha, beta; };

enum Epilogue { EpilogueNone = CUSYNC_EPILOGUE_NONE, EpilogueGeluErf = CUSYNC_EPILOGUE_GELU_ERF,
                EpilogueRelu = CUSYNC_EPILOGUE_RELU, EpilogueSiluMulDual = CUSYNC_EPILOGUE_SILU_MUL_DUAL };

// Tile grid of a GEMM the way CuSyncGemmHorizontalThreadblockSwizzle lays it
// out (gemm/threadblock/cusync_threadblock_swizzle.h:12-54): x = N tiles,
// y = M tiles, z = split-K slices.  Tile M of the sm_100a kernels is 128.
inline dim3 gemmGridShape(const GemmCoord& problem, int tileN, int splitK = 1) {
  return dim3((problem.n() + tileN - 1) / tileN, (problem.m() + 127) / 128, splitK);
}

template <typename CuStageT, int EpilogueKind = EpilogueNone, int TileN = 0>
class Gemm {
 public:
  static constexpr int kTileM = 128;

  struct Arguments {
    CuStageT custage;
    GemmCoord problem_size;
    TensorRef ref_A, ref_B, ref_C, ref_D;
    EpilogueParams epilogue;
    int split_k_slices;
    TensorRef ref_B2;   // second B operand of EpilogueSiluMulDual
    Arguments() : epilogue{1.0f, 0.0f}, split_k_slices(1) {}
    Arguments(CuStageT stage, GemmCoord problem, TensorRef a, TensorRef b, TensorRef c, TensorRef d,
              EpilogueParams epi = EpilogueParams{1.0f, 0.0f}, int splitK = 1, TensorRef b2 = TensorRef())
        : custage(stage), problem_size(problem), ref_A(a), ref_B(b), ref_C(c), ref_D(d), epilogue(epi),
          split_k_slices(splitK), ref_B2(b2) {}
  };

  // Public, as in the reference: callers increment params_.custage after a run.
  struct Params { CuStageT custage; } params_;

  Gemm() : plan_(nullptr) {}

  static Status can_implement(const Arguments& a) {
    if (a.split_k_slices < 1) return Status::kErrorNotSupported;
    if (a.split_k_slices > 1 && EpilogueKind == EpilogueSiluMulDual) return Status::kErrorNotSupported;
    if (a.epilogue.alpha != 1.0f || a.epilogue.beta != 0.0f) return Status::kErrorNotSupported;
    if (a.problem_size.m() <= 0 || a.problem_size.n() <= 0 || a.problem_size.k() <= 0)
      return Status::kErrorInvalidProblem;
    if (a.ref_A.ld % 8 || a.ref_B.ld % 8 || a.ref_D.ld % 8) return Status::kErrorMisalignedOperand;
    return Status::kSuccess;
  }

  static size_t get_workspace_size(const Arguments&) { return 0; }

  Status initialize(const Arguments& a, void* workspace = nullptr, cudaStream_t stream = nullptr) {
    (void)workspace; (void)stream;
    Status s = can_implement(a);
    if (s != Status::kSuccess) return s;
    destroy();
    params_.custage = a.custage;
    cusync_gemm_desc_t d{};
    d.m = a.problem_size.m(); d.n = a.problem_size.n(); d.k = a.problem_size.k();
    d.a = a.ref_A.ptr; d.lda = a.ref_A.ld;
    d.b = a.ref_B.ptr; d.ldb = a.ref_B.ld;
    d.b2 = a.ref_B2.ptr;
    d.d = a.ref_D.ptr; d.ldd = a.ref_D.ld;
    d.b_layout = CUSYNC_B_ROW_MAJOR_KN;
    d.epilogue = EpilogueKind;
    d.tile_n = TileN;
    d.max_ctas = 0;
    d.split_k = a.split_k_slices;   // explicit, as in the reference: the stage grid's z must match
    d.cta_pair = 0;
    d.stage = params_.custage.handle();
    int rc = cusync_gemm_plan_create(&plan_, &d);
    if (rc == CUSYNC_ERROR_UNSUPPORTED) return Status::kErrorNotSupported;
    return rc == CUSYNC_SUCCESS ? Status::kSuccess : Status::kErrorInternal;
  }

  Status update(const Arguments& a, void* workspace = nullptr) {
    (void)workspace;
    int rc = cusync_gemm_plan_update(plan_, a.ref_A.ptr, a.ref_B.ptr, a.ref_B2.ptr, a.ref_D.ptr);
    return rc == CUSYNC_SUCCESS ? Status::kSuccess : Status::kErrorInternal;
  }
  Status updateA(TensorRef a) { return cusync_gemm_plan_update(plan_, a.ptr, nullptr, nullptr, nullptr) == CUSYNC_SUCCESS ? Status::kSuccess : Status::kErrorInternal; }
  Status updateD(TensorRef d) { return cusync_gemm_plan_update(plan_, nullptr, nullptr, nullptr, d.ptr) == CUSYNC_SUCCESS ? Status::kSuccess : Status::kErrorInternal; }

  Status run(cudaStream_t stream = nullptr) {
    if (plan_ == nullptr) return Status::kErrorInternal;
    // The launch reads the run counter of the copy held in params_.
    if (params_.custage.handle()) cusync_stage_set_iter(params_.custage.handle(), params_.custage.currentIter());
    int rc = cusync_gemm_run(plan_, reinterpret_cast<cusync_stream_t>(stream));
    return rc == CUSYNC_SUCCESS ? Status::kSuccess : Status::kErrorInternal;
  }
  // Signature of the reference's overlapped launch; both of its branches
  // launch the same kernel (gemm/device/cusyncgemm.h:525-563).
  Status run(bool overlap, int* kernelExecuted, cudaStream_t stream = nullptr) {
    (void)overlap; (void)kernelExecuted;
    return run(stream);
  }
  Status operator()(cudaStream_t stream = nullptr) { return run(stream); }
  // The launch as a programmatic dependent of the producer kernel ahead of it in `stream`: in place of
  // prod.invokeWaitKernel(consumer_stream) and a second stream.  Consumers only.
  Status runDependent(cudaStream_t stream = nullptr) {
    if (plan_ == nullptr) return Status::kErrorInternal;
    if (params_.custage.handle()) cusync_stage_set_iter(params_.custage.handle(), params_.custage.currentIter());
    int rc = cusync_gemm_run_dependent(plan_, reinterpret_cast<cusync_stream_t>(stream));
    return rc == CUSYNC_SUCCESS ? Status::kSuccess : Status::kErrorInternal;
  }

  uint32_t numCtas() const { return cusync_gemm_plan_num_ctas(plan_); }
  void destroy() { if (plan_) { cusync_gemm_plan_destroy(plan_); plan_ = nullptr; } }

 private:
  cusync_gemm_plan_t* plan_;
};

}  // namespace b200
}  // namespace cusync
