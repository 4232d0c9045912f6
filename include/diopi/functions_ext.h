/*
 * Fused transformer-inference entry points (the "ext" family of DIOPI).
 *
 * None of these has a call site inside the reference tree: they are called by the external
 * DeepLinkExt package that the reference's CI pins (dipu/scripts/ci/ci_benchmark.sh:35,41).
 * The argument order follows the (ctx, outputs..., inputs..., attributes...) convention;
 * "signature unpinned" until diffed against upstream diopi/functions_ext.h.
 *
 * The arithmetic of each op is pinned by the reference's own CPU restatements:
 *   rms_norm    dicp/dicp/vendor/AscendGraph/ext_ops.py:47-49 and dicp/test/model/llama/model.py:34-39
 *   rotary_emb  dicp/dicp/vendor/AscendGraph/ext_ops.py:24-33 (half-split layout) and
 *               dicp/test/model/llama/model.py:58-69 (interleaved / complex layout)
 */
#ifndef DIOPI_FUNCTIONS_EXT_H_
#define DIOPI_FUNCTIONS_EXT_H_

#include "diopi/diopirt.h"

#ifdef __cplusplus
extern "C" {
#endif

/* out = input * rsqrt(mean(input^2 over normalized_shape) + eps) * weight (+ bias)
 * inv_rms (optional, may be NULL): the per-row rsqrt term, fp32 or the input dtype, shape [..., 1]. */
DIOPI_API diopiError_t diopiRMSNorm(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiTensorHandle_t inv_rms,
                                    diopiConstTensorHandle_t input, diopiSize_t normalized_shape, diopiConstTensorHandle_t weight,
                                    diopiConstTensorHandle_t bias, double eps);

/* Rotate feature pairs of x [..., seq, heads, dim] (or [tokens, heads, dim]) by the angle tables.
 * cos / sin: broadcastable to [..., seq, 1, dim/2] (half tables) or [..., seq, 1, dim] (full tables,
 * both halves equal). interleaved=false pairs (i, i+dim/2); interleaved=true pairs (2i, 2i+1).
 * conj=true rotates by the negative angle. out may alias x. */
DIOPI_API diopiError_t diopiRotaryEmbedding(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t x,
                                            diopiConstTensorHandle_t cos, diopiConstTensorHandle_t sin, const bool conj,
                                            const bool interleaved);

/* Fused scaled-dot-product attention (inference): out = softmax(scale * q k^T [+ causal mask]) v.
 * Fused form of the bmm / div / add(mask) / softmax / bmm sequence of dicp/test/model/llama/model.py:146-150; the
 * reference's CPU restatement of the fused operator is dicp/dicp/vendor/AscendGraph/ext_ops.py:52-86.
 * Prototype provisional ("signature unpinned": the DIOPI header is not part of the reference snapshot).
 * q [batch, seq_q, heads, dim]; k, v [batch, seq_kv, kv_heads, dim] with heads % kv_heads == 0 (grouped heads share
 * K / V); out like q; views with any pitches and a unit innermost pitch are taken as they are (no copies).
 * is_causal: key j is visible to query i iff j <= i + (seq_kv - seq_q). dropout_p must be 0, return_debug_mask false,
 * gen and debug_attn_mask NULL. softmax_lse: optional float32 [batch, heads, seq_q], log of the softmax denominator. */
DIOPI_API diopiError_t diopiMultiHeadAttention(diopiContextHandle_t ctx, diopiTensorHandle_t q, diopiTensorHandle_t k, diopiTensorHandle_t v,
                                               double dropout_p, bool is_causal, bool return_debug_mask, double scale, diopiTensorHandle_t out,
                                               diopiTensorHandle_t softmax_lse, diopiGeneratorHandle_t gen, diopiTensorHandle_t debug_attn_mask);

#ifdef __cplusplus
}
#endif
#endif /* DIOPI_FUNCTIONS_EXT_H_ */
