// Backward PLIF scan kernels with the modulation fused into the loads, f32 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_mod_bwd_f32(const BwdArgs& a) { return scan_mod_bwd_dispatch<float>(a); }
int scan_lin_bwd_f32(const BwdArgs& a) { return scan_lin_bwd_dispatch<float>(a); }
}  // namespace nsb
