/* flash_op_stubs.c -- TEST INFRASTRUCTURE.  The backend ops that the reference's graph files
 * reference for layers outside the attention path (Gated DeltaNet, MoE, hyper-connections, the
 * engram layer, sampling helpers).  flash_toy_gpu links the reference's graph code whole but
 * encodes only its attention layer, so these exist to satisfy the linker and stop the program if
 * one is ever reached.  (Declared without prototypes on purpose: this file does not include the
 * reference header, and none of them is ever called.) */
#include <stdio.h>
#include <stdlib.h>

#define STUB(name) void name(void) { fprintf(stderr, "flash_toy_gpu: %s is not part of the attention path\n", #name); abort(); }
STUB(qw_op_add_inplace) STUB(qw_op_embed_q4) STUB(qw_op_swiglu) STUB(qw_op_rms_norm_grouped) STUB(qw_op_qmm_q4_gather)
STUB(qw_op_qmv_q4_bank) STUB(qw_op_dmat_bf16) STUB(qw_op_qmv_q4_swiglu) STUB(qw_op_argmax_top2) STUB(qw_op_swiglu_split)
STUB(qw_op_silu_scale) STUB(qw_op_rms_norm_gated_sigmoid) STUB(qw_op_rms_norm_gated) STUB(qw_op_rms_norm_concat)
STUB(qw_op_repeat_cols) STUB(qw_op_qmv_q4_bank2) STUB(qw_op_ple_gate) STUB(qw_op_moe_route) STUB(qw_op_moe_group)
STUB(qw_op_moe_combine_shared) STUB(qw_op_hc_mix_up) STUB(qw_op_hc_mix) STUB(qw_op_hc_inject_norm) STUB(qw_op_hc_inject)
STUB(qw_op_gdn_gates) STUB(qw_op_gated_delta_prep) STUB(qw_op_gated_delta) STUB(qw_op_conv1d_dilated_silu)
STUB(qw_op_conv1d_causal_silu)
/* Only sizes a scratch buffer of the MoE layers at session creation (qwasar_flash_graph.c:122): an
 * upper bound for any tile height is one tile per pair plus one per expert. */
int qw_moe_max_tiles(int pairs, int experts) { return pairs + experts; }
void *qw_residency_new(void *bufs, int n) { (void)bufs; (void)n; return NULL; }
void qw_residency_free(void *r) { (void)r; }

