// TEST-ONLY translation unit (built by tests/test_gpu_bounded_waits.py, never linked into the library).
// Makes the kernels' bounded waits run out on purpose, the one way a wait failure may be provoked on a
// shared GPU: a flag that nothing sets, a limit of one millisecond, and a status word the host reads.
// No trap, no bad address, no endless loop; the context stays usable.
#define MOE_WAIT_LIMIT_NS 1000000ull   // 1 ms instead of the library's 0.4 s
#include "gemm_common.cuh"

namespace {

// The decode kernel's grid barrier with a target ONE ABOVE the number of CTAs that arrive.
__global__ void grid_barrier_probe(unsigned int* word2, int* status, unsigned int tag) {
  if (threadIdx.x != 0) return;
  if (blockIdx.x == 0) moe::grid_barrier_init(word2, tag);
  if (!moe::grid_barrier_tag_wait(word2, tag)) {
    atomicOr(status, 0x100);
    return;
  }
  moe::grid_barrier_arrive(word2);
  if (!moe::grid_barrier_wait(word2, tag, gridDim.x + 1)) atomicOr(status, moe::kErrGemm1Timeout);
}

// The pipeline's mbarrier wait on a phase that no arrival or TMA transaction ever completes; a second
// warp sees the CTA-wide abort flag and leaves as well.
__global__ void mbarrier_probe(int* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    moe::mbar_init(moe::smem_u32(&bar), 1);
    moe::fence_mbar_init();
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    if (!moe::mbar_wait(moe::smem_u32(&bar), 0, &abort_flag)) atomicOr(status, moe::kErrGemm2Timeout);
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag) atomicOr(status, 0x200);
}

}  // namespace

// status_dev: one int, zeroed by the caller; word_dev: two uints (any contents).  Returns the cudaError_t.
extern "C" int moe_test_wait_timeouts(int* status_dev, unsigned int* word_dev, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  grid_barrier_probe<<<4, 32, 0, stream>>>(word_dev, status_dev, 0x5EEDu);
  mbarrier_probe<<<1, 64, 0, stream>>>(status_dev);
  return static_cast<int>(cudaGetLastError());
}
