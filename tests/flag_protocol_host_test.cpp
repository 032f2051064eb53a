// Host model of the peer-memory flag protocols (csrc/flag_protocol.h): every rank is a thread, every rank's
// symmetric array an ordinary array, loads / stores are std::atomic acquire / release. Randomised delays change
// the arrival order on every round. Exit code 0 = all properties held.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <thread>
#include <vector>

#include "flag_protocol.h"

struct HostMem {
  static int load_acquire(const int* p) { return reinterpret_cast<const std::atomic<int>*>(p)->load(std::memory_order_acquire); }
  static void store_release(int* p, int v) { reinterpret_cast<std::atomic<int>*>(p)->store(v, std::memory_order_release); }
};

using namespace tlm::proto;

static std::atomic<int> g_fail{0};
#define CHECK(cond, ...) do { if (!(cond)) { if (g_fail.fetch_add(1) < 5) { fprintf(stderr, "FAILED %s: ", #cond); fprintf(stderr, __VA_ARGS__); fprintf(stderr, "\n"); } } } while (0)

static void jitter(std::mt19937& g, int max_us) {
  const int us = (int)(g() % (unsigned)(max_us + 1));
  if (us == 0) return;
  if (us < 3) std::this_thread::yield(); else std::this_thread::sleep_for(std::chrono::microseconds(us));
}

int main(int argc, char** argv) {
  const int n = argc > 1 ? atoi(argv[1]) : 4;
  const int rounds = argc > 2 ? atoi(argv[2]) : 2000;
  const unsigned seed = argc > 3 ? (unsigned)atoi(argv[3]) : 1u;
  const int start_epoch = argc > 4 ? atoi(argv[4]) : 0;          // e.g. 2147483000: the counters wrap during the run
  const int W = 16;                                              // words per parity for the scalar exchange
  const ReadyLayout L{16, 256, 272};
  const int buckets = 3, blocks = 5, bucket_words = 64;

  std::vector<std::vector<int>> flags(n, std::vector<int>(64, start_epoch));      // epoch exchange arrays
  std::vector<std::vector<float>> slots(n, std::vector<float>(2 * W, -1.f));     // parity slots of the scalar sum
  std::vector<std::vector<int>> ready(n, std::vector<int>(512, 0));
  std::vector<std::vector<int>> params(n, std::vector<int>(buckets * bucket_words * n, 0));   // every rank's replica
  std::vector<std::atomic<int>> entered(n);                                      // last exchange each rank entered
  for (auto& e : entered) e.store(start_epoch);
  std::vector<int*> flag_ptrs(n), ready_ptrs(n);
  for (int r = 0; r < n; ++r) { flag_ptrs[r] = flags[r].data(); ready_ptrs[r] = ready[r].data(); }

  auto rank_main = [&](int rank) {
    std::mt19937 g(seed * 7919u + (unsigned)rank);
    int epoch = start_epoch;
    for (int round = 0; round < rounds && g_fail.load() == 0; ++round) {
      // ---- 1 + 2: scalar sum with an epoch exchange and parity slots -------------------------------------
      epoch = (int)((unsigned)epoch + 1u);
      const float mine = (float)(round * 31 + rank);
      jitter(g, round % 7 == rank % 7 ? 40 : 2);                         // a different straggler every round
      for (int r = 0; r < n; ++r) slots[r][parity_slot(epoch, W, rank)] = mine;     // plain stores, ordered by the release below
      entered[rank].store(epoch, std::memory_order_relaxed);
      for (int r = 0; r < n; ++r) announce<HostMem>(flag_ptrs[r], rank, epoch);
      for (int r = 0; r < n; ++r) {
        while (!reached<HostMem>(flag_ptrs[rank] + r, epoch)) std::this_thread::yield();
        // property 1: rank r has entered exchange `epoch` (or a later one)
        CHECK(at_least(entered[r].load(std::memory_order_relaxed), epoch), "rank %d passed exchange %d before rank %d entered it", rank, epoch, r);
      }
      jitter(g, 3);
      float sum = 0.f, expect = 0.f;
      for (int r = 0; r < n; ++r) { sum += slots[rank][parity_slot(epoch, W, r)]; expect += (float)(round * 31 + r); }
      // property 2: nobody has overwritten this exchange's slots although fast ranks may already be in the next one
      CHECK(sum == expect, "rank %d round %d: sum %f != %f (a slot was overwritten early)", rank, round, sum, expect);

      // ---- 3: bucket updates published by the last of several "blocks", consumed through ready words -------
      for (int b = 0; b < buckets; ++b) {
        const int value = round * 1000 + b * 10 + rank + 1;
        std::vector<int> order(blocks);
        for (int i = 0; i < blocks; ++i) order[i] = i;
        std::shuffle(order.begin(), order.end(), g);
        for (int bi = 0; bi < blocks; ++bi) {
          const int blk = order[bi];
          // this block's share of my piece of bucket b, into every rank's replica (plain stores)
          for (int w = blk; w < bucket_words; w += blocks)
            for (int r = 0; r < n; ++r) params[r][(b * n + rank) * bucket_words + w] = value;
          std::atomic_thread_fence(std::memory_order_seq_cst);            // __threadfence_system
          const unsigned prev = (unsigned)reinterpret_cast<std::atomic<int>*>(&ready[rank][L.count0 + b])->fetch_add(1);
          publish_if_last<HostMem>(ready_ptrs.data(), n, rank, b, L, prev, (unsigned)blocks);
          jitter(g, 1);
        }
      }
      // next "forward pass": wait for every rank's update of each bucket, then read all pieces
      for (int b = 0; b < buckets; ++b) {
        const int expect_updates = HostMem::load_acquire(&ready[rank][L.epoch0 + b]);
        CHECK(expect_updates == round + 1, "rank %d: own update count %d in round %d", rank, expect_updates, round);
        for (int r = 0; r < n; ++r) {
          while (!ready_from<HostMem>(ready[rank].data(), b, L, r, expect_updates)) std::this_thread::yield();
          for (int w = 0; w < bucket_words; ++w) {
            const int v = params[rank][(b * n + r) * bucket_words + w];
            // property 3: every store of rank r's update is visible (a value from a LATER round is fine: r ran ahead)
            CHECK(v >= round * 1000 + b * 10 + r + 1, "rank %d reads stale word %d of bucket %d from rank %d: %d", rank, w, b, r, v);
          }
        }
      }
    }
  };
  std::vector<std::thread> th;
  for (int r = 0; r < n; ++r) th.emplace_back(rank_main, r);
  for (auto& t : th) t.join();
  if (g_fail.load()) { fprintf(stderr, "%d property violations\n", g_fail.load()); return 1; }
  printf("ok: %d ranks, %d rounds, seed %u, start epoch %d\n", n, rounds, seed, start_epoch);
  return 0;
}
