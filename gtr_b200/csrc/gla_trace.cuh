// Development builds only (-DGLA_TRACE): lane 0 of every warp of CTA 0 appends (clock << 8 | event id) to its own
// region of a buffer set with gla_b200_debug_set_trace; never part of the default library.
#pragma once
namespace gla { static unsigned long long* g_trace_buffer = nullptr; }
#define GLA_EV(id) do { if (blockIdx.x == 0 && P.trace != nullptr && (threadIdx.x & 31) == 0 && trace_n < 4096u) { \
        P.trace[(threadIdx.x >> 5) * 4096u + trace_n++] = ((unsigned long long)clock64() << 8) | (unsigned long long)(id); } } while (0)
extern "C" void gla_b200_debug_set_trace(void* p) { gla::g_trace_buffer = static_cast<unsigned long long*>(p); }
