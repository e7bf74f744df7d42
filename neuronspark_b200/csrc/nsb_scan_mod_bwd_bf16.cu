// Backward PLIF scan kernels with the modulation fused into the loads, bf16 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_mod_bwd_bf16(const BwdArgs& a) { return scan_mod_bwd_dispatch<__nv_bfloat16>(a); }
int scan_lin_bwd_bf16(const BwdArgs& a) { return scan_lin_bwd_dispatch<__nv_bfloat16>(a); }
}  // namespace nsb
