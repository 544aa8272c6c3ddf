// Host-side runtime shared by every entry point: last-error text, ABI version, and the
// driver entry point used to encode TMA tensor maps.
#include <stdio.h>
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

long long peer_wait_cycles();   // peer_combine.cu

// Host-side check and conversion of a caller's link description; false (with the error text set) when
// it is unusable.
bool make_link(const b200dsa_peer_link* in, PeerLinkDev* out, const char* who) {
  char msg[160];
  if (!in || !in->bufs || !in->state || in->world < 1 || in->world > kLinkMaxRanks || in->rank < 0 ||
      in->rank >= in->world || in->off_flags < 0 || (in->off_flags & 15) || in->slot < 1 || in->slot > 7 ||
      in->slot == 2) {
    snprintf(msg, sizeof(msg), "%s: bad peer link (1 <= world <= 8, slot 1 or 3..7, 16-byte aligned flags)", who);
    set_last_error(msg);
    return false;
  }
  for (int r = 0; r < in->world; ++r) {
    if (!in->bufs[r] || (reinterpret_cast<uintptr_t>(in->bufs[r]) & 15)) {
      snprintf(msg, sizeof(msg), "%s: every rank's buffer must be mapped and 16-byte aligned", who);
      set_last_error(msg);
      return false;
    }
    out->buf[r] = static_cast<unsigned char*>(in->bufs[r]);
  }
  out->rank = in->rank;
  out->world = in->world;
  out->off_flags = in->off_flags;
  out->slot = in->slot;
  out->state = in->state;
  out->wait_cycles = peer_wait_cycles();
  return true;
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
