// placeholder, replaced below
#include "context.h"
extern "C" {
uint64_t tnf_stack_record_bytes(uint32_t, uint32_t) { return 0; }
int32_t tnf_stack_create(tnf_ctx*, uint32_t, uint32_t, const tnf_stack_linear*, uint32_t, const uint32_t*, uint32_t, uint64_t, uint64_t, uint32_t, tnf_stack**) { return TNF_ERR_INVALID_ARGUMENT; }
int32_t tnf_stack_step(tnf_stack*, const uint64_t*, const uint64_t*, float) { return TNF_ERR_INVALID_ARGUMENT; }
int32_t tnf_stack_stats(tnf_stack*, uint64_t*) { return TNF_ERR_INVALID_ARGUMENT; }
int32_t tnf_stack_destroy(tnf_stack*) { return TNF_OK; }
}
