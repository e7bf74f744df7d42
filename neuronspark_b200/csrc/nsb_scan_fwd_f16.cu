// Forward PLIF scan kernels instantiated for the f16 stream dtype.
#include <cstring>

#include "nsb_scan.cuh"

namespace nsb {
int scan_fwd_f16(const FwdArgs& a) { return scan_fwd_dispatch<__half>(a); }
}  // namespace nsb
