// Placeholder until the tcgen05 kernel lands: reports the path as unavailable.
#include "scan.cuh"

namespace grmx {

bool scan_tcgen05_supported(const ScanParams&, int, int, const char** why) {
  *why = "tcgen05 kernel not built";
  return false;
}

int launch_scan_tcgen05(const ScanParams&, cudaStream_t) {
  return fail(GRMX_ERR_UNSUPPORTED, "tcgen05 kernel not built");
}

}  // namespace grmx
