// Forward PLIF scan kernels with the modulation fused into the loads, and the row-parameter
// scan with the binary residual applied to its spikes, f16 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_mod_fwd_f16(const FwdArgs& a) { return scan_mod_fwd_dispatch<__half>(a); }
int scan_res_fwd_f16(const FwdArgs& a) { return scan_res_fwd_dispatch<__half>(a); }
int scan_pat_fwd_f16(const FwdArgs& a) { return scan_pat_fwd_dispatch<__half>(a); }
int scan_lin_fwd_f16(const FwdArgs& a) { return scan_lin_fwd_dispatch<__half>(a); }
}  // namespace nsb
