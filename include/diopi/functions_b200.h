/*
 * Entry points of libdiopi_impl.so that are additions of this implementation, not part of DIOPI.
 */
#ifndef DIOPI_FUNCTIONS_B200_H_
#define DIOPI_FUNCTIONS_B200_H_

#include "diopi/diopirt.h"
#include "dipu_b200/peer_space.h"

#ifdef __cplusplus
extern "C" {
#endif

/* No counterpart in the reference. Health word of the tensor-core kernels on the current device: 0 while no bounded
 * device-side wait has ever timed out, 1 afterwards, -1 if it cannot be read. Synchronises the device. */
DIOPI_API int diopiB200GemmStatus(void);

/* No counterpart in the reference. One-time set-up on the current device for hosts that want it out of the first operator
 * call: allocates and clears the tensor-core kernels' status word (otherwise a cudaMalloc and a synchronising memset inside
 * the first matrix product on that device). Call it where the host initialises a device; repeated calls are free. */
DIOPI_API diopiError_t diopiB200Init(void);

/* No counterpart in the reference.
 *
 * Matrix product for callers that are not allowed to allocate device memory at the moment of the call: code running
 * while a framework's allocator lock is held or inside an allocator callback, a host whose memory pool is frozen
 * (fixed-budget serving processes), or a thread that must not enter the driver's allocation path. diopiMm obtains the
 * tensor-core kernel's status word with cudaMalloc on first use; this variant keeps that scratch in a 256-byte
 * static __device__ block inside the library instead (every GPU that loads the library holds those 256 bytes until
 * exit) and calls no cudaMalloc / cudaFree / host-allocator routine.
 *
 *   out  [m, n]  row pitch ldo            (elements)
 *   mat1 [m, k]  row pitch ld1, k contiguous
 *   mat2 [n, k]  row pitch ld2 when mat2_is_nk != 0 (a weight in nn.Linear layout: out = mat1 * mat2^T),
 *        [k, n]  row pitch ld2 otherwise
 *   dtype: diopi_dtype_bfloat16 or diopi_dtype_float16 for all three; fp32 accumulation.
 * Pointers must be 16-byte aligned and pitches multiples of 8 elements (the TMA rules); anything else, and any
 * dimension outside [1, 2^31), is rejected with diopiErrorOccurred and a message, never served by another path.
 * The scratch need of this kernel does not grow with the problem, so the static block is always enough.
 *
 * The first call on a device looks up the block's device address, and the first call of each tile variant on a device (the
 * variant depends on the problem's shape) raises that kernel's shared-memory limit; make a first call of every shape you
 * will use before any stream capture. Every call clears the status word on `stream` before the kernel runs and all calls share
 * the block, which keeps the last call's value: calls that overlap on the GPU (different streams) race on it, so
 * serialise them. diopiB200NoAllocStatus() reads the word back (synchronises). */
DIOPI_API diopiError_t diopiB200MmNoAlloc(diopiStreamHandle_t stream, void* out, const void* mat1, const void* mat2, int64_t m, int64_t n,
                                          int64_t k, int64_t ld1, int64_t ld2, int mat2_is_nk, int64_t ldo, diopiDtype_t dtype);
DIOPI_API int diopiB200NoAllocStatus(void);

/* No counterpart in the reference, where a row-parallel linear is diopiMm followed by an all-reduce of its result
 * (ProcessGroupDICL::allreduce, dipu/torch_dipu/csrc_dipu/runtime/distributed/ProcessGroupDICL.cpp:539-567).
 *
 * input [M, K] x mat2 [K, N] (bfloat16 or float16, the layouts diopiMm takes on its tensor-core path) is this rank's
 * partial sum. Nothing is stored locally: the kernel's epilogue writes every 32 x 256 piece into staging slot `slot` of
 * the rank that owns the piece's rows (rank r owns rows [r * M / nranks, (r + 1) * M / nranks)) over peer memory and
 * raises the piece's ready flag with `epoch`, while later tiles are still being multiplied. b200_dicl_peer_reduce_gather
 * (include/dipu_b200/vendor_c_api.h), called next with the same slot and epoch on every rank, sums the pieces and
 * distributes the result. `epoch` must grow from call to call and be the same on every rank; `prev_epoch` is the epoch of
 * the previous call that used `slot` (0 if none): the kernel does not overwrite a peer's slot before that call's
 * reduction has finished there (bounded wait; a time-out raises diopiB200GemmStatus).
 * M must be a multiple of 256 and of 128 * nranks, N a multiple of 256, M * N elements must fit a slot.
 * diopiB200SetPushWaitLimitNs: limit of that wait for the launches that follow (0 = the default of 2 s). */
DIOPI_API diopiError_t diopiB200MmPush(diopiContextHandle_t ctx, diopiConstTensorHandle_t input, diopiConstTensorHandle_t mat2,
                                       const b200PeerSpace* space, int32_t slot, uint32_t epoch, uint32_t prev_epoch);
DIOPI_API void diopiB200SetPushWaitLimitNs(unsigned long long ns);

/* Fused steps of a decode iteration. No counterparts among the reference's call sites, which dispatch the pieces one by one
 * (dicp/test/model/llama/model.py:34-39 RMSNorm, :58-69 rotary, :134-138 cache append, :174-175 SwiGLU, :193-201 residual
 * adds); every function rounds where the separate calls round unless stated, so a model can switch call by call.
 *
 * diopiB200MmSwiGLU    out [M, F] = silu(input @ gate) * (input @ up) for mat2 [K, 2F] whose columns 2j and 2j+1 are the gate
 *                      and up weights of feature j (interleave w1 / w3 once at load time; the nn.Linear layout [2F, K] is
 *                      passed as its transposed view). One product, the SiLU and the multiplication in its epilogue, formed in
 *                      fp32 and rounded ONCE (the separate calls round the two products, the SiLU and the product again).
 *                      bfloat16 / float16, 1 to 128 rows.
 * diopiB200AddRMSNorm  sum_out = input + residual (rounded like diopiAdd), norm_out = RMSNorm(sum_out) * weight (weight may be
 *                      NULL): the residual add that ends one block and the norm that opens the next, in one pass.
 *                      [rows, cols] bfloat16 / float16, inputs with contiguous rows, dense outputs.
 * diopiB200RopeAppendKV  from qkv [B, (Hq + 2 Hkv) * D], the output of ONE projection over the concatenated q / k / v weight:
 *                      q rotated -> q_out [B, Hq, D]; k rotated -> k_cache[:, :, position, :]; v -> v_cache[:, :, position, :]
 *                      (caches [B, Hkv, L, D] with any pitches). Half-split rotary layout (pairs i, i + D/2), cos / sin float32
 *                      [1 or B, D / 2] (row b % rows), products and sums in fp32 rounded once like diopiRotaryEmbedding. */
DIOPI_API diopiError_t diopiB200MmSwiGLU(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input,
                                         diopiConstTensorHandle_t mat2);
DIOPI_API diopiError_t diopiB200AddRMSNorm(diopiContextHandle_t ctx, diopiTensorHandle_t sum_out, diopiTensorHandle_t norm_out,
                                           diopiConstTensorHandle_t input, diopiConstTensorHandle_t residual, diopiConstTensorHandle_t weight,
                                           double eps);
DIOPI_API diopiError_t diopiB200RopeAppendKV(diopiContextHandle_t ctx, diopiTensorHandle_t q_out, diopiConstTensorHandle_t qkv,
                                             diopiConstTensorHandle_t cos, diopiConstTensorHandle_t sin, diopiTensorHandle_t k_cache,
                                             diopiTensorHandle_t v_cache, int64_t position);

#ifdef __cplusplus
}
#endif
#endif /* DIOPI_FUNCTIONS_B200_H_ */
