// Forward PLIF scan kernels instantiated for the f32 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_fwd_f32(const FwdArgs& a) { return scan_fwd_dispatch<float>(a); }
}  // namespace nsb
