// Backward PLIF scan kernels with the modulation fused into the loads, f16 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_mod_bwd_f16(const BwdArgs& a) { return scan_mod_bwd_dispatch<__half>(a); }
int scan_lin_bwd_f16(const BwdArgs& a) { return scan_lin_bwd_dispatch<__half>(a); }
}  // namespace nsb
