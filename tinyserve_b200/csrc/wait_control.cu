// The one switch over every translation unit's bounded-wait settings (bounded_wait.cuh): each unit
// that waits on mbarriers registers a setter for its own constants when the library is loaded, and
// ts_set_wait_control calls them all. Upstream's analogue of a failed wait is a hard error on the
// host (src/tinyserve/engine.py:173-175); here a kernel that gives up leaves a code that the engine
// raises on.
namespace ts {
typedef int (*WaitControlSetter)(long long, int);    // as in bounded_wait.cuh
}

namespace {
constexpr int MAX_UNITS = 16;
ts::WaitControlSetter g_setters[MAX_UNITS];   // zero-initialised before any unit registers
int g_num_setters;
}  // namespace

extern "C" void ts_wait_control_register(ts::WaitControlSetter setter) {
  for (int i = 0; i < g_num_setters; ++i)
    if (g_setters[i] == setter) return;
  if (g_num_setters < MAX_UNITS) g_setters[g_num_setters++] = setter;
}

// cycles: the bound of every mbarrier wait, in clock cycles (<= 0: the default, about a second).
// unarmed: non-zero makes every kernel skip its copies and their expect-tx (tests only).
// Applies to the current device; call with nothing of this library in flight. Returns 0 or a cudaError_t.
extern "C" int ts_set_wait_control(long long cycles, int unarmed) {
  if (cycles <= 0) cycles = 2000000000ll;
  for (int i = 0; i < g_num_setters; ++i) {
    const int rc = g_setters[i](cycles, unarmed);
    if (rc != 0) return rc;
  }
  return 0;
}

extern "C" int ts_wait_control_units() { return g_num_setters; }
