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

#ifdef __cplusplus
}
#endif
#endif /* DIOPI_FUNCTIONS_EXT_H_ */
