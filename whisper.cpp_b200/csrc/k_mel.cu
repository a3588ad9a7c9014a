// log-mel front-end (placeholder until the kernel lands)
#include "b200_common.cuh"
extern "C" int b200_log_mel(int, const float *, int64_t, const float *, int, float *, int64_t, int *, int *) { return B200_ERR_ARG; }
