// Model / state / token-loop entry points of the C ABI (include/pyre_b200.h).
#include "pb_internal.h"

#include <stdio.h>

#define PB_TODO(name) PB_FAIL((pb_ctx*)nullptr, PB_UNSUPPORTED, name)

extern "C" {
int pb_model_create(pb_ctx*, const pb_cfg*, pb_model**) { return PB_UNSUPPORTED; }
int pb_model_set_tensor(pb_model*, int, int, pb_qmat*) { return PB_UNSUPPORTED; }
int pb_model_set_vec(pb_model*, int, int, const float*, int64_t) { return PB_UNSUPPORTED; }
int pb_model_finalize(pb_model*, int, int) { return PB_UNSUPPORTED; }
int pb_model_destroy(pb_model*) { return PB_UNSUPPORTED; }
int pb_state_create(pb_model*, int, pb_state**) { return PB_UNSUPPORTED; }
int pb_state_destroy(pb_state*) { return PB_UNSUPPORTED; }
int pb_state_fill_kv(pb_state*, int, int, const float*, const float*, int64_t) { return PB_UNSUPPORTED; }
int pb_state_fill_kv_synth(pb_state*, int, int64_t, uint64_t) { return PB_UNSUPPORTED; }
int pb_state_set_pos(pb_state*, int64_t) { return PB_UNSUPPORTED; }
int pb_state_pos(const pb_state*, int64_t*) { return PB_UNSUPPORTED; }
int pb_forward(pb_state*, const uint32_t*, int, float*) { return PB_UNSUPPORTED; }
int pb_step_greedy(pb_state*, const uint32_t*, uint32_t*) { return PB_UNSUPPORTED; }
int pb_decode_greedy(pb_state*, const uint32_t*, int, uint32_t*) { return PB_UNSUPPORTED; }
int pb_verify(pb_state*, const uint32_t*, int, float*) { return PB_UNSUPPORTED; }
int pb_keep(pb_state*, int, int) { return PB_UNSUPPORTED; }
int pb_draft(pb_state*, int, uint32_t*, int*) { return PB_UNSUPPORTED; }
int pb_state_snapshot(pb_state*, void*, size_t*) { return PB_UNSUPPORTED; }
int pb_state_restore(pb_state*, const void*, size_t) { return PB_UNSUPPORTED; }
int pb_caps_get(const pb_model*, pb_caps*) { return PB_UNSUPPORTED; }
int pb_stats_get(const pb_state*, pb_stats*) { return PB_UNSUPPORTED; }
int pb_moe_forward(pb_state*, int, const float*, int, float*, int32_t*) { return PB_UNSUPPORTED; }
int pb_deltanet_step(pb_state*, int, const float*, float*) { return PB_UNSUPPORTED; }
int pb_attn_step(pb_state*, int, const float*, float*) { return PB_UNSUPPORTED; }
int pb_state_get_lin(pb_state*, int, float*, float*) { return PB_UNSUPPORTED; }
int pb_state_set_lin(pb_state*, int, const float*, const float*) { return PB_UNSUPPORTED; }
int pb_kv4_pack(pb_ctx*, const float*, int64_t, uint32_t*, float*) { return PB_UNSUPPORTED; }
int pb_kv4_unpack(pb_ctx*, const uint32_t*, const float*, int64_t, float*) { return PB_UNSUPPORTED; }
}
