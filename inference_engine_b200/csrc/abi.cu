// Version and error-string entry points of the b200kv C ABI.
#include "b200kv.h"

#include <atomic>

namespace b200kv {
static std::atomic<int> g_chained{0};
bool chained_launch_enabled() { return g_chained.load(std::memory_order_relaxed) != 0; }
}  // namespace b200kv

extern "C" void b200kv_set_chained_launch(int enabled) { b200kv::g_chained.store(enabled ? 1 : 0, std::memory_order_relaxed); }
extern "C" int b200kv_get_chained_launch(void) { return b200kv::chained_launch_enabled() ? 1 : 0; }

extern "C" int b200kv_version(void) { return B200KV_VERSION; }

extern "C" const char* b200kv_error_string(int code) {
  switch (code) {
    case B200KV_OK: return "ok";
    case B200KV_E_NULL: return "a required pointer is NULL";
    case B200KV_E_SHAPE: return "unsupported geometry (head_dim must be 128, Hq a multiple of Hkv with ratio <= 8, page_size a multiple of 16 when paged)";
    case B200KV_E_ALIGN: return "pointer or stride not aligned (bf16 rows need 8-byte, q/out of decode attention 16-byte alignment)";
    case B200KV_E_WORKSPACE: return "workspace too small (see b200kv_decode_attn_workspace_bytes)";
    case B200KV_E_LAUNCH: return "CUDA launch failed";
    case B200KV_E_RANGE: return "size argument out of range";
    case B200KV_E_STATIC_LIMIT: return "this batch needs more scratch than the 8 MiB built into the library: use b200kv_decode_attn with a caller workspace";
    default: return "unknown b200kv error";
  }
}
