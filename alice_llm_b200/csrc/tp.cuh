// Tensor-parallel helpers (csrc/tp.cu).
#pragma once
#include <stddef.h>

struct alice_engine;

namespace alice {

// In-place all-gather over the engine's group, queued on the engine's stream: every rank has written its
// own bytes_per_rank bytes at base + rank * bytes_per_rank; afterwards all ranks hold all world * bytes_per_rank
// bytes. No-op for a group of one.
int tp_all_gather(alice_engine* e, void* base, size_t bytes_per_rank);
// Destroys the communicator (engine teardown).
void tp_release(alice_engine* e);

}  // namespace alice
