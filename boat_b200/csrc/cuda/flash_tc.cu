#include "common.cuh"
namespace boatcu {
bool attn_tc_supported(int, int64_t, int64_t, int64_t, int) { return false; }
int attn_fwd_tc(int, int64_t, int64_t, int64_t, int, float, const void*, const void*, const void*, int, void*, float*) { return set_error(99, "no tc"); }
size_t attn_bwd_tc_scratch_bytes(int, int64_t, int64_t, int64_t) { return 0; }
int attn_bwd_tc(int, int64_t, int64_t, int64_t, int, float, const void*, const void*, const void*, const void*, const float*, const float*, int, void*, void*, void*, void*, size_t) { return set_error(99, "no tc"); }
}
