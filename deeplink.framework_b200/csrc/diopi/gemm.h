// Internal description of one (batched) matrix product and the kernels that can run it.
#pragma once

#include "common.h"

struct CUtensorMap_st;  // the driver API's tensor-map descriptor (cuda.h)
struct b200PeerSpace;   // dipu_b200/peer_space.h

namespace b200 {

// C[b,m,n] = alpha * sum_k A[b,m,k] * B[b,k,n] + beta * bias[b,m,n]; all strides in elements.
struct GemmProblem {
    int64_t batch = 1, M = 0, N = 0, K = 0;
    const void* A = nullptr;
    int64_t a_sb = 0, a_sm = 0, a_sk = 0;
    const void* B = nullptr;
    int64_t b_sb = 0, b_sk = 0, b_sn = 0;
    void* C = nullptr;
    int64_t c_sb = 0, c_sm = 0, c_sn = 0;
    const void* bias = nullptr;  // optional; strides may be 0 (broadcast)
    int64_t bias_sb = 0, bias_sm = 0, bias_sn = 0;
    diopiDtype_t ab_dtype = diopi_dtype_unsupported;
    diopiDtype_t c_dtype = diopi_dtype_unsupported;
    diopiDtype_t bias_dtype = diopi_dtype_unsupported;
    float alpha = 1.f, beta = 0.f;
    // Status word to report into; nullptr = the per-device word the library allocates on first use.
    uint32_t* status_override = nullptr;
    // Epilogue of the single-row-block (M <= 128) kernel. kSwiGLU: the N columns of the product are (gate, up) pairs,
    // columns 2j and 2j+1; C is [M, N / 2] and receives silu(gate_j) * up_j, formed in fp32 and rounded once.
    enum Epilogue { kPlain = 0, kSwiGLU = 1 };
    int epilogue = kPlain;
};

// tcgen05 / TMEM / TMA kernel (bf16 or fp16 operands, fp32 accumulation).
bool gemm_tc_eligible(const GemmProblem& g);
diopiError_t gemm_tc_launch(const GemmProblem& g, cudaStream_t stream);

// CTA-pair variant (cta_group::2, 256 x 256 tiles) for large products; gemm_tc_launch hands over to it when it applies.
bool gemm_tc2_applies(const GemmProblem& g);
diopiError_t gemm_tc2_launch(const GemmProblem& g, cudaStream_t stream);

// The CTA-pair kernel with a pushing epilogue: g.C is ignored, every 32 x 256 piece of the product goes to the staging slot
// of the rank that owns its rows (dipu_b200/peer_space.h) and raises that piece's ready flag with `epoch`.
diopiError_t gemm_tc2_push_launch(const GemmProblem& g, const ::b200PeerSpace& space, int slot, uint32_t epoch, uint32_t prev_epoch,
                                  cudaStream_t stream);

// Shared by the tensor-core translation units.
bool tc_encode_map(::CUtensorMap_st* map, diopiDtype_t dtype, const void* base, int64_t inner, int64_t rows, int64_t batch, int64_t row_pitch_elems,
                   int64_t batch_pitch_elems, int box_rows);
// dims = {inner, d1, d2, d3} (innermost first), pitch_elems = pitches of d1, d2, d3; box = {128 bytes, box1, box2, 1}.
bool tc_encode_map4(::CUtensorMap_st* map, diopiDtype_t dtype, const void* base, const int64_t dims[4], const int64_t pitch_elems[3], int box1,
                    int box2);
uint32_t* tc_status_word();
// Raises a kernel's dynamic shared-memory limit once per (device, kernel); safe to call from concurrent threads.
cudaError_t tc_ensure_smem_attr(const void* kernel, int bytes);
// Limit of the pushing kernel's wait for the permission to overwrite a peer's staging slot (0 = the default of 2 s).
void gemm_tc2_set_push_wait_limit_ns(unsigned long long ns);

// Fused attention (attention.cu).
bool attention_prefill_applies(const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& out);
diopiError_t attention_prefill_launch(const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& out, const TensorView* lse,
                                      bool causal, double scale, cudaStream_t stream);

bool attention_decode_applies(const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& out);
diopiError_t attention_decode_launch(diopiContextHandle_t ctx, const TensorView& q, const TensorView& k, const TensorView& v, const TensorView& out,
                                     const TensorView* lse, double scale, cudaStream_t stream);

}  // namespace b200
