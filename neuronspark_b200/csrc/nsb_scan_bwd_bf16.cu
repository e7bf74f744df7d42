// Backward PLIF scan kernels instantiated for the bf16 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_bwd_bf16(const BwdArgs& a) { return scan_bwd_dispatch<__nv_bfloat16>(a); }
}  // namespace nsb
