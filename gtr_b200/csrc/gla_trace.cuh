// Development builds only (-DGLA_TRACE): lane 0 of every warp of three CTAs appends (value << 8 | event id) to its own
// region of a buffer set with gla_b200_debug_set_trace; never part of the default library.
#pragma once
namespace gla { static unsigned long long* g_trace_buffer = nullptr; }
#define GLA_EVV(id, val) do { if (blockIdx.x % 60 == 0 && P.trace != nullptr && (threadIdx.x & 31) == 0 && trace_n < 4096u) { \
        P.trace[((blockIdx.x / 60) * 20 + (threadIdx.x >> 5)) * 4096u + trace_n++] = ((unsigned long long)(val) << 8) | (unsigned long long)(id); } } while (0)
#define GLA_EV(id) GLA_EVV(id, clock64())
extern "C" void gla_b200_debug_set_trace(void* p) { gla::g_trace_buffer = static_cast<unsigned long long*>(p); }
