// Status strings and build identification.
#include "flagattn_b200.h"

extern "C" const char *fa_status_string(int status) {
  switch (status) {
    case FA_OK: return "ok";
    case FA_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or bad enum)";
    case FA_ERR_UNSUPPORTED: return "unsupported head size, dtype or group size";
    case FA_ERR_ALIGNMENT: return "pointer or stride is not 16-byte aligned";
    case FA_ERR_LAUNCH: return "CUDA launch failed";
    case FA_ERR_WORKSPACE: return "workspace pointer missing or too small";
    case FA_ERR_TOO_LARGE: return "request exceeds a fixed built-in capacity";
  }
  return "unknown status";
}

extern "C" const char *fa_version(void) { return "flagattn_b200 1 sm_100a"; }
