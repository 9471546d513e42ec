// Internal view of the peer-group objects for the providers (the C types are opaque outside
// peer_group.cpp).
#pragma once

#include "kernels.hpp"
#include "loom_b200.h"

namespace lb {

// The signal block of the group as the last kernel of a gathering command needs it.
PeerSignal peer_signal_of(const lb_peer_group *group, long long wait_cycles);
// Device array [world] of the addresses, in this process, of every rank's copy of the buffer.
void *const *peer_buffer_table(const lb_peer_buffer *buffer);
int peer_group_device(const lb_peer_group *group);
int peer_group_clock_khz(const lb_peer_group *group);

} // namespace lb
