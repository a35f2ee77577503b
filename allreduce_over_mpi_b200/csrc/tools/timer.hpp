// Host stopwatch with integer readouts, the role of the reference's newplan::Timer
// (cost_model/timer.h:12-132, vector_add/time_record.h:6-126).  One class instead of two
// near-identical copies; steady clock; fractional readouts are available too.
#pragma once
#include <chrono>
#include <cstdint>

namespace ft {
class Timer {
 public:
  void Start() { t0_ = clock::now(); running_ = true; }
  void Stop() { t1_ = clock::now(); running_ = false; }
  int64_t NanoSeconds() const { return std::chrono::duration_cast<std::chrono::nanoseconds>(end() - t0_).count(); }
  int64_t MicroSeconds() const { return NanoSeconds() / 1000; }
  int64_t MilliSeconds() const { return NanoSeconds() / 1000000; }
  int64_t Seconds() const { return NanoSeconds() / 1000000000; }
  double seconds() const { return NanoSeconds() * 1e-9; }
 private:
  using clock = std::chrono::steady_clock;
  clock::time_point end() const { return running_ ? clock::now() : t1_; }
  clock::time_point t0_{}, t1_{};
  bool running_ = false;
};
}  // namespace ft
