// Forward PLIF scan kernels with the modulation fused into the loads, and the row-parameter
// scan with the binary residual applied to its spikes, f32 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_mod_fwd_f32(const FwdArgs& a) { return scan_mod_fwd_dispatch<float>(a); }
int scan_res_fwd_f32(const FwdArgs& a) { return scan_res_fwd_dispatch<float>(a); }
int scan_pat_fwd_f32(const FwdArgs& a) { return scan_pat_fwd_dispatch<float>(a); }
int scan_lin_fwd_f32(const FwdArgs& a) { return scan_lin_fwd_dispatch<float>(a); }
}  // namespace nsb
