#include "launchers.h"
namespace alg {
bool head_tcgen05_supports(const HeadParams&) { return false; }
int head_tcgen05_splits(int, int) { return 1; }
int launch_head_tcgen05(const HeadParams&, cudaStream_t) { set_error("not built"); return ALG_ERR_UNSUPPORTED; }
}
