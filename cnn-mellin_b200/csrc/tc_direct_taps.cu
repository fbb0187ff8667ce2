// The tensor-core forward / grad-input kernel built for layers with many linear
// taps: weights of all taps do not fit a pipeline stage, so every block of rows
// is staged once per group of four taps.  Same source as tc_direct.cu; the
// macro selects the tap-group variants of its loops and plan.
#define MELLIN_TAP_GROUPS 1
#include "tc_direct.cu"
