// A stand-in for libgdrapi for tests without the gdrdrv kernel module: "pinning" accepts any address and the "BAR1
// window" is the memory itself, so a test can hand GdrWindow a host buffer and check the pointer arithmetic (the pinned range
// starts at a 64 KB boundary below the address) and the ordered store.
// Build: g++ -shared -fPIC fake_gdrapi.cc -o libfake_gdrapi.so
#include <cstddef>
#include <cstdint>
#include <cstdlib>

extern "C" {

struct gdr_mh {
  unsigned long h;
};
struct gdr_info {
  uint64_t va;
  uint64_t mapped_size;
  uint32_t page_size;
  uint64_t tm_cycles;
  uint32_t cycles_per_ms;
  unsigned mapped : 1;
  unsigned wc_mapping : 1;
  int mapping_type;
};

static int g_open = 0;
static int g_pins = 0;

void* gdr_open(void) {
  g_open++;
  return &g_open;
}
int gdr_close(void*) {
  g_open--;
  return 0;
}
int gdr_pin_buffer(void*, unsigned long addr, size_t size, uint64_t, uint32_t, gdr_mh* handle) {
  if ((addr & 0xffff) != 0 || size == 0 || (size & 0xffff) != 0) return 22;
  handle->h = addr;
  g_pins++;
  return 0;
}
int gdr_unpin_buffer(void*, gdr_mh) {
  g_pins--;
  return 0;
}
int gdr_map(void*, gdr_mh handle, void** va, size_t) {
  *va = reinterpret_cast<void*>(handle.h);
  return 0;
}
int gdr_unmap(void*, gdr_mh, void*, size_t) { return 0; }
int gdr_get_info(void*, gdr_mh handle, gdr_info* info) {
  info->va = handle.h;
  info->mapped_size = 65536;
  info->page_size = 65536;
  info->mapped = 1;
  info->wc_mapping = 0;
  return 0;
}
int fake_gdr_live_pins(void) { return g_pins; }

}  // extern "C"
