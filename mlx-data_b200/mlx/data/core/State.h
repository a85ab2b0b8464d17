// Random state shared by every op that draws parameters
// (mlx/data/core/State.h:14-23): one process-wide generator, copied into a
// thread-local state the first time a thread draws after a set_state().
#pragma once

#include <cstdint>
#include <memory>
#include <random>

namespace mlx {
namespace data {
namespace core {

struct State {
  std::mt19937 randomGenerator;
  int64_t version = 0;
};

// The calling thread's state.
std::shared_ptr<State> get_state();

// Reseed the process-wide generator; call from the main thread only.
void set_state(int64_t seed);

} // namespace core
} // namespace data
} // namespace mlx
