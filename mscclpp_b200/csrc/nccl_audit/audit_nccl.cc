// rtld-audit library: with LD_AUDIT=libmscclpp_b200_audit_nccl.so every attempt of the dynamic linker to load
// libnccl.so / libnccl.so.2 (a DT_NEEDED entry or a dlopen) is answered with the NCCL-API shim of this package.
// Unlike LD_PRELOAD this also redirects programs that dlopen NCCL by name at run time. The shim must be findable by
// the linker (LD_LIBRARY_PATH or an absolute path in MSCCLPP_B200_NCCL_SHIM).
// (The reference ships the same mechanism: src/ext/nccl/audit-shim/audit_nccl.cc:9-17.)
#include <link.h>

#include <cstdlib>
#include <cstring>

extern "C" __attribute__((visibility("default"))) unsigned int la_version(unsigned int) { return LAV_CURRENT; }

extern "C" __attribute__((visibility("default"))) char* la_objsearch(const char* name, uintptr_t*, unsigned int) {
  const char* base = std::strrchr(name, '/');
  base = base ? base + 1 : name;
  if (std::strcmp(base, "libnccl.so.2") != 0 && std::strcmp(base, "libnccl.so") != 0) return const_cast<char*>(name);
  const char* shim = std::getenv("MSCCLPP_B200_NCCL_SHIM");
  return const_cast<char*>(shim != nullptr && shim[0] != '\0' ? shim : "libmscclpp_b200_nccl.so");
}
