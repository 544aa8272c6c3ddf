// Host-side runtime shared by every entry point: last-error text, ABI version, and the
// driver entry point used to encode TMA tensor maps.
#include <stdlib.h>
#include <string.h>

#include "b200dsa_common.cuh"

namespace b200dsa {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* msg) {
  strncpy(g_last_error, msg ? msg : "", sizeof(g_last_error) - 1);
  g_last_error[sizeof(g_last_error) - 1] = 0;
}

PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !ptr) {
    set_last_error("cuTensorMapEncodeTiled is not available from this driver");
    return nullptr;
  }
  fn = reinterpret_cast<PFN_encodeTiled>(ptr);
  return fn;
}

bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("B200DSA_PDL");
    on = (e && e[0] == '1') ? 1 : 0;
  }
  return on != 0;
}

}  // namespace b200dsa

extern "C" int b200dsa_abi_version(void) { return 1; }
extern "C" const char* b200dsa_last_error(void) { return b200dsa::g_last_error; }
