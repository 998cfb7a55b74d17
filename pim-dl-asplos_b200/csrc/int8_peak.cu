// Measured int8 tensor rate of this GPU: the denominator for the tensor-side roofline of the tcgen05
// LUT kernel.  Runs nothing but tcgen05.mma kind::i8 (128 x N x 32 per instruction, int32 accumulators
// in tensor memory, operand A in tensor memory, operand B one shared-memory tile that is never
// reloaded), four issuing warps per CTA, one CTA per SM, and reports the time by CUDA events and the
// cycles of one CTA by its own clock, so the caller gets both TOPS and multiply-adds per clock per SM.
// Operand values do not matter (zeros).  Every wait is bounded.
#include "kernels.h"
#include "ptx.cuh"

namespace lutamm {

namespace {

constexpr uint32_t kPeakWarps = 4;

template <uint32_t N>
__global__ void __launch_bounds__(kPeakWarps * 32, 1) int8_peak_kernel(uint32_t slabs, unsigned long long* cycles_out, uint32_t* dev_err) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint32_t s_tmem;
    __shared__ uint32_t s_abort;
    __shared__ uint64_t s_bar[kPeakWarps];
    __shared__ long long s_end[kPeakWarps];
    for (uint32_t i = threadIdx.x; i < N * 128 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (uint32_t w = 0; w < kPeakWarps; ++w) mbar_init(smem_u32(&s_bar[w]), 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x < 32) { tmem_alloc(smem_u32(&s_tmem), 512); tmem_relinquish(); }
    tc_fence_before_sync();
    fence_proxy_async_smem();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = s_tmem, warp = threadIdx.x >> 5;
    volatile uint32_t* abort_word = &s_abort;
    constexpr uint32_t idesc = umma_idesc_i8(128, N, 1, 1);
    const uint64_t b_desc = umma_desc_k_sw128(smem_u32(smem));
    const long long t0 = clock64();
    for (uint32_t i = warp; i < slabs; i += kPeakWarps) {
        if (elect_one()) {
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk)  // A: 8 columns per 32 bytes of K, behind the accumulator
                umma_i8_ts(tmem, tmem + N + (i & 3u) * 32 + 8 * kk, b_desc + 2 * kk, idesc, 1u);
        }
        __syncwarp();
    }
    if (elect_one()) umma_commit(smem_u32(&s_bar[warp]));
    __syncwarp();
    mbar_wait(smem_u32(&s_bar[warp]), 0, abort_word);
    s_end[warp] = clock64();
    __syncthreads();
    if (threadIdx.x == 0) {
        long long e = s_end[0];
        for (uint32_t w = 1; w < kPeakWarps; ++w) e = s_end[w] > e ? s_end[w] : e;
        if (blockIdx.x == 0) *cycles_out = (unsigned long long)(e - t0);
        if (s_abort) atomicExch(dev_err, 3u);
    }
    if (threadIdx.x < 32) { tc_fence_after_sync(); tmem_dealloc(tmem, 512); }
}

}  // namespace

cudaError_t launch_int8_peak(uint32_t n_tile, uint32_t slabs, uint32_t grid, unsigned long long* d_cycles, uint32_t* dev_err,
                             cudaStream_t s, const char** why) {
    *why = nullptr;
    // more than half an SM's shared memory: never two of these CTAs (512 tensor-memory columns each) on one SM
    const size_t smem = 120 * 1024;
    cudaError_t e;
    if (n_tile == 256) {
        if ((e = cudaFuncSetAttribute(int8_peak_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        int8_peak_kernel<256><<<grid, kPeakWarps * 32, smem, s>>>(slabs, d_cycles, dev_err);
    } else if (n_tile == 192) {
        if ((e = cudaFuncSetAttribute(int8_peak_kernel<192>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        int8_peak_kernel<192><<<grid, kPeakWarps * 32, smem, s>>>(slabs, d_cycles, dev_err);
    } else if (n_tile == 128) {
        if ((e = cudaFuncSetAttribute(int8_peak_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
        int8_peak_kernel<128><<<grid, kPeakWarps * 32, smem, s>>>(slabs, d_cycles, dev_err);
    } else {
        *why = "int8 peak measurement: N tile must be 128, 192 or 256";
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}


// ---- self-test of the way out after a wait that runs out -----------------------------------------
// One CTA sets up what the tcgen05 LUT kernel sets up (tensor memory, an mbarrier), then one thread waits
// - with the library's own bounded wait, limited to `polls` probes - on a barrier nobody ever arrives at.
// The wait gives up, the abort word is set, the CTA goes through the same tear-down as the LUT kernel
// (report in the device error word, everybody meets, tensor memory is freed) and returns.  Nothing traps and
// nothing spins on: the host reads the error word and the context stays usable.
namespace {
__global__ void __launch_bounds__(128, 1) stalled_wait_kernel(uint32_t polls, uint32_t* dev_err) {
    __shared__ uint32_t s_tmem;
    __shared__ uint32_t s_abort;
    __shared__ uint64_t s_bar;
    if (threadIdx.x == 0) {
        s_abort = 0;
        mbar_init(smem_u32(&s_bar), 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x < 32) { tmem_alloc(smem_u32(&s_tmem), 32); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    volatile uint32_t* abort_word = &s_abort;
    if (threadIdx.x == 32) (void)mbar_wait_limited(smem_u32(&s_bar), 0, abort_word, polls);   // phase 0 never completes
    __syncthreads();
    if (*abort_word && threadIdx.x == 0) atomicExch(dev_err, 4u);
    __syncthreads();
    if (threadIdx.x < 32) { tc_fence_after_sync(); tmem_dealloc(s_tmem, 32); }
}
}  // namespace

cudaError_t launch_stalled_wait(uint32_t polls, uint32_t* dev_err, cudaStream_t s) {
    stalled_wait_kernel<<<1, 128, 0, s>>>(polls, dev_err);
    return cudaGetLastError();
}

}  // namespace lutamm
