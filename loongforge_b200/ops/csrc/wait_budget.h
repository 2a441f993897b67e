// Run-time budget of the waits on flags that ANOTHER GPU writes (fused tensor-parallel GEMMs, expert-parallel
// exchange, peer-memory optimizer). It is separate from the compile-time budget of the waits inside one CTA's
// own pipeline (LF_WAIT_BUDGET_CYCLES, about a second): a healthy pipeline stage completes in microseconds,
// whereas a peer rank that writes a checkpoint, evaluates or stalls on its data loader is legitimately late by
// many seconds. Every wait stays bounded; a wait that runs out sets LF_ERR_WAIT_PEER in the status word.
#pragma once

namespace lf {

// SM clock cycles; the conversion from time assumes 2 GHz (the part's maximum is 1.965 GHz, so a budget never
// expires early). Default two minutes. One value per process, read at every launch.
inline long long g_peer_wait_cycles = 120ll * 2000000000ll;

inline void set_peer_wait_budget_ms(double ms) {
  if (ms < 0.001) ms = 0.001;
  g_peer_wait_cycles = static_cast<long long>(ms * 2.0e6);
}
inline double peer_wait_budget_ms() { return static_cast<double>(g_peer_wait_cycles) / 2.0e6; }

}  // namespace lf
