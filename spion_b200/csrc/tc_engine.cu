// placeholder replaced below
#include "common.cuh"
bool tc_engine_supports(const spion_ctx*) { return false; }
int tc_engine_prepare(spion_ctx*) { return SPION_OK; }
void tc_engine_release(spion_ctx*) {}
int tc_engine_forward(spion_ctx*, const void*, const void*, const void*, const float*, void*, void*) { return SPION_ERR_UNSUPPORTED; }
int tc_engine_backward(spion_ctx*, const void*, const void*, const void*, const void*, const void*, const void*, void*, float*, void*, void*, void*) { return SPION_ERR_UNSUPPORTED; }
