#include "mlx/data/core/State.h"

#include <mutex>

namespace mlx {
namespace data {
namespace core {

namespace {
State& process_state() {
  static State s;
  return s;
}
std::mutex& process_mutex() {
  static std::mutex m;
  return m;
}
} // namespace

void set_state(int64_t seed) {
  std::lock_guard<std::mutex> g(process_mutex());
  State& s = process_state();
  s.randomGenerator = std::mt19937(seed);
  s.version++;
}

std::shared_ptr<State> get_state() {
  static thread_local std::shared_ptr<State> mine;
  std::lock_guard<std::mutex> g(process_mutex());
  const State& s = process_state();
  if (!mine || mine->version != s.version) {
    mine = std::make_shared<State>(s);
  }
  return mine;
}

} // namespace core
} // namespace data
} // namespace mlx
