#include "common.cuh"
bool attention_tc_supported(const AttnArgs&) { return false; }
int attention_fwd_tc(const AttnArgs&, cudaStream_t) { return femto_fail(FEMTO_ERR_UNSUPPORTED, "tcgen05 attention not built"); }
int attention_bwd_tc(const AttnArgs&, cudaStream_t) { return femto_fail(FEMTO_ERR_UNSUPPORTED, "tcgen05 attention not built"); }
size_t attention_bwd_tc_ws_bytes(int, int, int, int) { return 0; }
