// Flag protocols of the peer-memory kernels, written once for the device and for a host test.
//
// The kernels in collectives.cu synchronise ranks through int32 words in symmetric memory. Three small protocols
// are used; each is a template over a memory policy `Mem` that supplies
//     static int  load_acquire(const int* p);        // ld.acquire.sys on the device, atomic acquire load on the host
//     static void store_release(int* p, int v);      // st.release.sys                 atomic release store
// so that the same code runs inside the CUDA kernels (DeviceMem, common.cuh) and in a host program in which
// every rank is a thread and the "peers' memories" are ordinary arrays (tests/flag_protocol_host_test.cpp). The
// host test drives them with randomised arrival orders and delays and checks the properties stated below.
//
//  1. epoch exchange   word [r] of rank d's array is written only by rank r and read only by rank d. Exchange
//                      number e: every rank stores e into its word on every peer, then waits until all words of
//                      its own array have reached e. Property: no rank passes exchange e before every rank has
//                      entered it. Epochs only grow, comparisons are wrap-safe (signed difference).
//  2. parity slots     a value exchanged together with epoch e lives in slot (e & 1): a fast rank that is already
//                      in exchange e + 1 writes the other slot, so the value of e cannot be overwritten before a
//                      slow rank has read it (it can only be overwritten in e + 2, which no rank can enter before
//                      every rank has left e + 1, i.e. has long read e).
//  3. ready words      word [bucket][r] of every rank is written by rank r after ALL of its stores of that bucket
//                      (block counter: the block that completes the count publishes). A consumer that sees all n
//                      words at its own update count may read the bucket. Property: it then sees every store.
#pragma once

#ifdef __CUDACC__
#define TLM_HD __host__ __device__ __forceinline__
#else
#define TLM_HD inline
#endif

namespace tlm {
namespace proto {

// true once `value` has reached `epoch`. The difference is taken in unsigned arithmetic: a signed subtraction that
// overflows when the counters wrap is undefined, and compilers do turn `a - b >= 0` into `a >= b`.
TLM_HD bool at_least(int value, int epoch) { return (int)((unsigned int)value - (unsigned int)epoch) >= 0; }

// true once the word has reached `epoch` (wrap-safe)
template <class Mem>
TLM_HD bool reached(const int* word, int epoch) {
  return at_least(Mem::load_acquire(word), epoch);
}

// rank `rank` announces `epoch` to peer r: word [rank] of r's array
template <class Mem>
TLM_HD void announce(int* peer_array, int rank, int epoch) {
  Mem::store_release(peer_array + rank, epoch);
}

// slot of a value that travels with exchange `epoch` (see 2. above); `width` values per parity
TLM_HD int parity_slot(int epoch, int width, int index) { return (epoch & 1) * width + index; }

// ready words: layout of one rank's array
struct ReadyLayout {
  int stride;       // words per bucket (>= number of ranks)
  int epoch0;       // first of the per-bucket "updates done by this rank" words
  int count0;       // first of the per-bucket "blocks finished" counters
};

// Called by one thread of a block after the block's stores are fenced. `prev` is the value the block's atomic
// increment of the bucket's counter returned. Returns true for the block that completes the count; that block
// resets the counter and publishes the next update count to every rank.
template <class Mem>
TLM_HD bool publish_if_last(int* const* arrays, int n, int rank, int bucket, const ReadyLayout& L, unsigned int prev,
                            unsigned int blocks) {
  if (prev != blocks - 1) return false;
  int* mine = arrays[rank];
  Mem::store_release(mine + L.count0 + bucket, 0);
  const int done = (int)((unsigned int)Mem::load_acquire(mine + L.epoch0 + bucket) + 1u);
  for (int r = 0; r < n; ++r) Mem::store_release(arrays[r] + bucket * L.stride + rank, done);
  Mem::store_release(mine + L.epoch0 + bucket, done);
  return true;
}

// consumer side: has rank r's update number `expect` of `bucket` arrived in this rank's array?
template <class Mem>
TLM_HD bool ready_from(const int* mine, int bucket, const ReadyLayout& L, int r, int expect) {
  return reached<Mem>(mine + bucket * L.stride + r, expect);
}

}  // namespace proto
}  // namespace tlm
