// Tuning aid, compiled only with -DMELLIN_TUNING_HOOKS (not part of the public ABI).
// Per-role cycle counters of block 0 of the last tensor-core forward /
// grad-input launch (mellin_tc_profile) or weight-gradient launch
// (mellin_tc_gradw_profile) made while the environment variable
// MELLIN_TC_PROFILE was "1": out[2 * r] = cycles role r spent waiting on
// barriers, out[2 * r + 1] = cycles it spent working; r = 0 epilogue,
// 1 converter, 2 MMA issuer, 3 copy issuer (the weight-gradient kernel adds
// r = 4, its second converter group, out[12] = MMA cycles spent waiting for
// the level-1 accumulators, out[13] = stages).  16 values.
#pragma once
#ifdef MELLIN_TUNING_HOOKS
extern "C" int mellin_tc_profile(long long *out);
extern "C" int mellin_tc_gradw_profile(long long *out);
#endif
