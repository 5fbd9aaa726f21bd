// Development builds only (-DGLA_TRACE): lane 0 of every warp of the CTAs that take work items 5, 53 and 101 first
// appends (value << 8 | event id) to its own region of a buffer set with gla_b200_debug_set_trace; never part of the
// default library.
#pragma once
namespace gla { static unsigned long long* g_trace_buffer = nullptr; }
#define GLA_TRACE_PICK(item) do { if (trace_slot == -2) trace_slot = (item) == 5 ? 0 : (item) == 53 ? 1 : (item) == 101 ? 2 : -1; } while (0)
#define GLA_EVV(id, val) do { if (trace_slot >= 0 && P.trace != nullptr && (threadIdx.x & 31) == 0 && trace_n < 4096u) { \
        P.trace[(trace_slot * 20 + (threadIdx.x >> 5)) * 4096u + trace_n++] = ((unsigned long long)(val) << 8) | (unsigned long long)(id); } } while (0)
#define GLA_EV(id) GLA_EVV(id, clock64())
extern "C" void gla_b200_debug_set_trace(void* p) { gla::g_trace_buffer = static_cast<unsigned long long*>(p); }
