// The tensor-core forward kernel with the epilogue the reference's models apply
// around a layer fused in: y = mask * relu(layer(x)) for per-utterance lengths
// along the linear axis, and no work at all for tiles past an utterance's end.
// Same source as tc_direct.cu; the macro selects the masked tile test and store.
#define MELLIN_MASKED 1
#include "tc_direct.cu"
