// Backward PLIF scan kernels instantiated for the f32 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_bwd_f32(const BwdArgs& a) { return scan_bwd_dispatch<float>(a); }
}  // namespace nsb
