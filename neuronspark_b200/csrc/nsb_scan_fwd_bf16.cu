// Forward PLIF scan kernels instantiated for the bf16 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_fwd_bf16(const FwdArgs& a) { return scan_fwd_dispatch<__nv_bfloat16>(a); }
}  // namespace nsb
