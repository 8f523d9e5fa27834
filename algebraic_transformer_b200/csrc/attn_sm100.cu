#include "launchers.h"
namespace alg {
bool attn_tcgen05_supports(const AttnParams&, int) { return false; }
int launch_attn_tcgen05(const AttnParams&, cudaStream_t) { set_error("not built"); return ALG_ERR_UNSUPPORTED; }
}
