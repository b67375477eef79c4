// flag_protocol.h -- host model of the flag protocol of the peer-memory kernels, for tests with threads as ranks.
//
// The device kernels (csrc/kernels/comm_kernels.cu, the gated GEMM in gemm_sm100.cu) synchronise ranks with 64-bit
// flags in symmetric memory: flag[s] on rank d is written only by rank s, with a release store of a monotonically
// increasing epoch; a waiter spins with acquire loads until the flag reaches the epoch it expects, for a bounded
// time, and reports {who waited, on whom, expected, seen} instead of spinning on.  Nothing is ever reset, so a
// kernel sequence can be replayed.  This header states the same rules with std::atomic so that the protocol itself
// (not the CUDA code) can be exercised deterministically on the host, with a rank that stops signalling.
#pragma once
#include <atomic>
#include <chrono>
#include <cstdint>
#include <memory>
#include <thread>
#include <vector>

namespace ff {
namespace flagproto {

struct WaitReport {
  bool ok = true;
  int waiter = -1, peer = -1;
  uint64_t expected = 0, seen = 0;
};

class FlagBoard {
public:
  FlagBoard(int ranks, int slots) : ranks_(ranks), slots_(slots), flags_(new std::atomic<uint64_t>[(size_t)ranks * ranks * slots]) {
    for (size_t i = 0; i < (size_t)ranks * ranks * slots; ++i) flags_[i].store(0, std::memory_order_relaxed);
  }
  int ranks() const { return ranks_; }
  // rank `src` raises its flag `slot` on rank `dst`
  void signal(int src, int dst, int slot, uint64_t epoch) { at(dst, src, slot).store(epoch, std::memory_order_release); }
  // rank `me` waits until `peer`'s flag `slot` (in me's memory) has reached `target`
  WaitReport bounded_wait(int me, int peer, int slot, uint64_t target, std::chrono::nanoseconds limit) const {
    const auto t0 = std::chrono::steady_clock::now();
    WaitReport r;
    for (;;) {
      const uint64_t v = at(me, peer, slot).load(std::memory_order_acquire);
      if (v >= target) return r;
      if (std::chrono::steady_clock::now() - t0 > limit) {
        r.ok = false; r.waiter = me; r.peer = peer; r.expected = target; r.seen = v;
        return r;
      }
      std::this_thread::yield();
    }
  }
  // the barrier of signal_wait_kernel: signal every peer, then wait for every peer
  WaitReport barrier(int me, int slot, uint64_t epoch, std::chrono::nanoseconds limit) {
    for (int p = 0; p < ranks_; ++p) signal(me, p, slot, epoch);
    for (int p = 0; p < ranks_; ++p) {
      WaitReport r = bounded_wait(me, p, slot, epoch, limit);
      if (!r.ok) return r;
    }
    return WaitReport{};
  }

private:
  std::atomic<uint64_t> &at(int owner, int writer, int slot) const { return flags_[((size_t)owner * ranks_ + writer) * slots_ + slot]; }
  int ranks_, slots_;
  std::unique_ptr<std::atomic<uint64_t>[]> flags_;
};

struct RankResult {
  uint64_t epochs_done = 0;
  WaitReport report;
  uint64_t checksum = 0;  // sum over epochs of the values published by the peers that this rank read after each barrier
  double seconds = 0;
};

// `ranks` threads run `epochs` rounds of: publish a value, barrier, read every peer's value, barrier.  Rank
// `silent_rank` (if >= 0) stops taking part after `silent_after` epochs without signalling again -- the host form of a
// rank that left.  Every wait is bounded by `limit_ms`.
inline std::vector<RankResult> run_rounds(int ranks, int epochs, int silent_rank, int silent_after, int limit_ms) {
  FlagBoard board(ranks, 2);
  std::vector<std::atomic<uint64_t>> data(ranks);
  for (auto &d : data) d.store(0);
  std::vector<RankResult> out(ranks);
  std::vector<std::thread> threads;
  const auto limit = std::chrono::milliseconds(limit_ms);
  for (int r = 0; r < ranks; ++r) {
    threads.emplace_back([&, r] {
      const auto t0 = std::chrono::steady_clock::now();
      for (int e = 1; e <= epochs; ++e) {
        if (r == silent_rank && e > silent_after) break;
        data[r].store((uint64_t)e * 1000 + r, std::memory_order_relaxed);   // ordered before the flag by its release store
        WaitReport w = board.barrier(r, 0, (uint64_t)e, limit);
        if (!w.ok) { out[r].report = w; break; }
        for (int p = 0; p < ranks; ++p) out[r].checksum += data[p].load(std::memory_order_relaxed);
        w = board.barrier(r, 1, (uint64_t)e, limit);                           // nobody overwrites before everyone has read
        if (!w.ok) { out[r].report = w; break; }
        out[r].epochs_done = (uint64_t)e;
      }
      out[r].seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    });
  }
  for (auto &t : threads) t.join();
  return out;
}

}  // namespace flagproto
}  // namespace ff
