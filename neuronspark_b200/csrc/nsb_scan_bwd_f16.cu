// Backward PLIF scan kernels instantiated for the f16 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_bwd_f16(const BwdArgs& a) { return scan_bwd_dispatch<__half>(a); }
}  // namespace nsb
