/* abi_check.c -- compile-time proof that include/cwick_compat.h lays the
 * boundary structs out exactly as the reference's header does. Built (not run)
 * by `make ref` with the reference's src/ on the include path. TEST
 * INFRASTRUCTURE ONLY. */
#include <stddef.h>

#include "cwick.h"
#define CWICK_COMPAT_TYPES_ONLY
#include "../include/cwick_compat.h"

#define SAME_SIZE(a, b) _Static_assert(sizeof(a) == sizeof(b), "size of " #a)
#define SAME_OFF(a, b, f) _Static_assert(offsetof(a, f) == offsetof(b, f), "offset of " #f)

SAME_SIZE(cwick_error, cwkc_error);
SAME_OFF(cwick_error, cwkc_error, message);
SAME_SIZE(cwick_tensor, cwkc_tensor);
SAME_OFF(cwick_tensor, cwkc_tensor, kind);
SAME_OFF(cwick_tensor, cwkc_tensor, data);
SAME_OFF(cwick_tensor, cwkc_tensor, scales);
SAME_OFF(cwick_tensor, cwkc_tensor, name);
SAME_SIZE(cwick_model_spec, cwkc_model_spec);
SAME_OFF(cwick_model_spec, cwkc_model_spec, hidden_size);
SAME_OFF(cwick_model_spec, cwkc_model_spec, num_attention_heads);
SAME_OFF(cwick_model_spec, cwkc_model_spec, q_lora_rank);
SAME_OFF(cwick_model_spec, cwkc_model_spec, kv_lora_rank);
SAME_OFF(cwick_model_spec, cwkc_model_spec, qk_nope_head_dim);
SAME_OFF(cwick_model_spec, cwkc_model_spec, qk_rope_head_dim);
SAME_OFF(cwick_model_spec, cwkc_model_spec, value_head_dim);
SAME_OFF(cwick_model_spec, cwkc_model_spec, rms_norm_eps_f);
SAME_OFF(cwick_model_spec, cwkc_model_spec, linear_num_heads);
SAME_OFF(cwick_model_spec, cwkc_model_spec, linear_head_dim);
SAME_OFF(cwick_model_spec, cwkc_model_spec, short_conv_kernel_size);
SAME_OFF(cwick_model_spec, cwkc_model_spec, gate_lower_bound);
SAME_OFF(cwick_model_spec, cwkc_model_spec, layers);
SAME_OFF(cwick_model_spec, cwkc_model_spec, quant);
SAME_OFF(cwick_model_spec, cwkc_model_spec, index_head_dim);
SAME_OFF(cwick_model_spec, cwkc_model_spec, index_n_heads);
SAME_OFF(cwick_model_spec, cwkc_model_spec, index_topk);
SAME_OFF(cwick_model_spec, cwkc_model_spec, index_kpool);
SAME_OFF(cwick_model_spec, cwkc_model_spec, n_sparse_layers);
SAME_SIZE(cwick_indexer_weights, cwkc_indexer_weights);
SAME_SIZE(cwick_indexer_state, cwkc_indexer_state);
SAME_OFF(cwick_indexer_state, cwkc_indexer_state, n_pools);
_Static_assert((int)CWICK_WEIGHT_BF16 == (int)CWKC_WEIGHT_BF16 && (int)CWICK_WEIGHT_F32 == (int)CWKC_WEIGHT_F32 &&
               (int)CWICK_WEIGHT_FP8_E4M3 == (int)CWKC_WEIGHT_FP8_E4M3, "weight kinds");
_Static_assert((int)CWICK_ERR_UNSUPPORTED == (int)CWK_ERR_UNSUPPORTED && (int)CWICK_ERR_ARGUMENT == (int)CWK_ERR_ARGUMENT &&
               (int)CWICK_ERR_MEMORY == (int)CWK_ERR_MEMORY && (int)CWICK_ERR_STATE == (int)CWK_ERR_STATE, "status codes");
int cwk_abi_check_ok = 1;
