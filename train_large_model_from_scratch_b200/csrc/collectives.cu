// Gradient reduce-scatter and fused AdamW + parameter all-gather over NVLink
// peer memory (one process per GPU, buffers in symmetric memory).
//
//   reduce_scatter : each rank sums ITS slice of the flat fp32 gradient buffer (or of its
//                    bf16 rounding, the "bf16 wire") over all ranks, reading the peers' buffers directly
//                    (multimem.ld_reduce through the NVSwitch when a multicast
//                    mapping is given, else one P2P load per peer), and emits
//                    per-block sum-of-squares partials for the global grad norm.
//   adamw_gather   : clipped AdamW on the rank's slice (fp32 master, exp_avg,
//                    exp_avg_sq) whose bf16 result is stored straight into every
//                    rank's parameter replica (multimem.st or P2P stores), i.e.
//                    the all-gather rides on the optimizer's store.
//   peer_barrier   : flag exchange; also fused as the prologue of reduce_scatter.
//
// Flags live in a symmetric int32 array: slot r of rank d is written only by
// rank r (st.release.sys) and polled only by rank d (ld.acquire.sys). Waits are
// bounded (2 s); on a timeout the kernel records a status code, skips its
// remote accesses and returns.
#include "common.cuh"

namespace tlm {

constexpr int MAX_PEERS = 16;

struct PeerPtrs {
  void* p[MAX_PEERS];
};

// Threads 0..n-1 of the calling block: (optionally) publish `epoch` to every
// peer, then wait until every peer has published it here. Returns false on timeout.
__device__ __forceinline__ bool flag_exchange(const PeerPtrs& flags, int rank, int n, int epoch, bool do_signal,
                                              unsigned int* status, unsigned int site) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < n) {
    const int r = threadIdx.x;
    if (do_signal) {
      __threadfence_system();
      proto::announce<DeviceMem>(reinterpret_cast<int*>(flags.p[r]), rank, epoch);
    }
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + r;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!proto::reached<DeviceMem>(mine, epoch)) {
      if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > kWaitLimitNs) {
        report_status(status, (site << 8) | (unsigned int)r);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// Epochs. Every exchange on a flag array uses the next integer. A caller may pass it (epoch > 0) or let the
// kernels count themselves (epoch == 0): word EPOCH_SLOT of the rank's OWN flag array holds the last epoch used,
// read at kernel start and advanced by the kernel (or its single-block follow-up) at the end. All ranks run the
// same sequence of exchanges, so their counters agree, and since no launch argument changes from step to step
// the launches can be recorded in a CUDA graph and replayed.
constexpr int EPOCH_SLOT = 32;
__device__ __forceinline__ int resolve_epoch(const PeerPtrs& flags, int rank, int epoch) {
  return epoch > 0 ? epoch : (int)((unsigned int)reinterpret_cast<volatile int*>(flags.p[rank])[EPOCH_SLOT] + 1u);
}
__device__ __forceinline__ void commit_epoch(const PeerPtrs& flags, int rank, int epoch_arg, int epoch_used) {
  if (epoch_arg <= 0) reinterpret_cast<volatile int*>(flags.p[rank])[EPOCH_SLOT] = epoch_used;
}

__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int n, int epoch_arg, unsigned int* status) {
  const int epoch = resolve_epoch(flags, rank, epoch_arg);
  flag_exchange(flags, rank, n, epoch, true, status, 40);
  if (threadIdx.x == 0) commit_epoch(flags, rank, epoch_arg, epoch);
}

// Sum of one fp32 value over the ranks: each rank stores its value into slot `rank` of every peer's `slots`
// array (symmetric memory, n floats), a flag exchange follows, then every rank adds the n slots in rank order
// (so all ranks get the same bits). One block of >= n threads. Slots are double-buffered by epoch parity: a
// fast rank's next store cannot overwrite a value a slow rank has not summed yet.
__global__ void peer_allreduce_scalar_kernel(PeerPtrs slots, PeerPtrs flags, const float* __restrict__ in, float* __restrict__ out,
                                             float scale, int rank, int n, int epoch_arg, unsigned int* status) {
  const int epoch = resolve_epoch(flags, rank, epoch_arg);
  const int par = proto::parity_slot(epoch, MAX_PEERS, 0);
  if ((int)threadIdx.x < n) reinterpret_cast<volatile float*>(slots.p[threadIdx.x])[par + rank] = *in;
  const bool ok = flag_exchange(flags, rank, n, epoch, true, status, 44);
  if (threadIdx.x == 0) {
    float acc = 0.f;
    if (ok) {
      const volatile float* mine = reinterpret_cast<const volatile float*>(slots.p[rank]) + par;
      for (int r = 0; r < n; ++r) acc += mine[r];
    }
    *out = acc * scale;
    commit_epoch(flags, rank, epoch_arg, epoch);
  }
}

// Waits until *flag >= expect or `limit_ns` elapse; a timeout is reported through the status word
// (site 42) and the kernel returns normally, so the context and the stream stay usable.
__global__ void wait_flag_kernel(const int* flag, int expect, unsigned long long limit_ns, unsigned int* status) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!proto::reached<DeviceMem>(flag, expect)) {
    if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > limit_ns) {
      report_status(status, (42u << 8) | 1u);
      break;
    }
  }
}

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b32x4(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// out[i] = sum_r grads[r][lo + i],  i in [0, len).  partials[blockIdx.x] = sum out[i]^2 over the block's share.
// Prologue: every block waits until all ranks have published `epoch` (their
// backward pass, which precedes this kernel in stream order, is complete).
__global__ void reduce_scatter_kernel(PeerPtrs grads, const float* mc_grads, PeerPtrs flags, float* __restrict__ out,
                                      float* __restrict__ partials, long long lo, long long len, int rank, int n,
                                      int epoch_arg, unsigned int* status) {
  __shared__ float red[32];
  const bool ok = flag_exchange(flags, rank, n, resolve_epoch(flags, rank, epoch_arg), blockIdx.x == 0, status, 41);
  float acc = 0.f;
  if (ok) {
    const long long nvec = len / 4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
      float4 s;
      if (mc_grads != nullptr) {
        s = multimem_ld_reduce_f32x4(mc_grads + lo + i * 4);
      } else {
        s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < n; ++r) {
          const int src = (rank + r) % n;                      // start at self, spread the peers
          const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[src]) + lo + i * 4);
          s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
      }
      reinterpret_cast<float4*>(out)[i] = s;
      acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) partials[blockIdx.x] = v;
  }
}

// bf16 wire format: every rank first rounds its fp32 gradients into a symmetric bf16 staging buffer
// (cast_bf16_kernel, local), then each rank sums ITS slice over all ranks' staging buffers with fp32
// accumulation. Half the NVLink bytes of the fp32 wire at the price of one rounding of each addend
// (and, through the switch, of the sum: multimem.ld_reduce returns bf16 for bf16 operands).
__global__ void cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long nvec = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(src)[2 * i], b = reinterpret_cast<const float4*>(src)[2 * i + 1];
    reinterpret_cast<uint4*>(dst)[i] = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
  }
}

__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const __nv_bfloat16* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

__global__ void reduce_scatter_bf16_kernel(PeerPtrs wire, const __nv_bfloat16* mc_wire, PeerPtrs flags, float* __restrict__ out,
                                           float* __restrict__ partials, long long lo, long long len, int rank, int n,
                                           int epoch_arg, unsigned int* status) {
  __shared__ float red[32];
  const bool ok = flag_exchange(flags, rank, n, resolve_epoch(flags, rank, epoch_arg), blockIdx.x == 0, status, 43);
  float acc = 0.f;
  if (ok) {
    const long long nvec = len / 8;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
      float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (mc_wire != nullptr) {
        const uint4 v = multimem_ld_reduce_bf16x8(mc_wire + lo + i * 8);
        const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), d = unpack_bf16(v.w);
        s[0] = a.x; s[1] = a.y; s[2] = b.x; s[3] = b.y; s[4] = c.x; s[5] = c.y; s[6] = d.x; s[7] = d.y;
      } else {
        for (int r = 0; r < n; ++r) {
          const int src = (rank + r) % n;
          const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(wire.p[src]) + lo + i * 8);
          const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), d = unpack_bf16(v.w);
          s[0] += a.x; s[1] += a.y; s[2] += b.x; s[3] += b.y; s[4] += c.x; s[5] += c.y; s[6] += d.x; s[7] += d.y;
        }
      }
      reinterpret_cast<float4*>(out)[2 * i] = make_float4(s[0], s[1], s[2], s[3]);
      reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(s[4], s[5], s[6], s[7]);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc += s[k] * s[k];
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) partials[blockIdx.x] = v;
  }
}

// Also advances the self-counted epoch of the reduce-scatter that ran before it (all of whose blocks read it).
__global__ void sum_partials_kernel(const float* __restrict__ partials, int n, float* __restrict__ out, PeerPtrs flags,
                                    int rank, int epoch_arg) {
  __shared__ double red[32];
  double acc = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += (double)partials[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
    out[0] = (float)t;
    if (epoch_arg <= 0) commit_epoch(flags, rank, epoch_arg, resolve_epoch(flags, rank, epoch_arg));
  }
}

// AdamW on [0, len) of the shard; bf16 result goes to element lo + i of every rank's replica.
__global__ void adamw_gather_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                    const float* __restrict__ g, PeerPtrs params, __nv_bfloat16* mc_params,
                                    const float* __restrict__ scale_ptr, long long lo, long long len, int rank, int n,
                                    float lr, float beta1, float beta2, float eps, float wd, float inv_bc1,
                                    float inv_sqrt_bc2, const float* __restrict__ hyper, PeerPtrs ready, int bucket) {
  if (hyper != nullptr) { lr = hyper[0]; inv_bc1 = hyper[1]; inv_sqrt_bc2 = hyper[2]; }   // per-step values from device memory
  const float scale = *scale_ptr;
  const long long nvec = len / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float pa[8], ma[8], va[8], ga[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 a = reinterpret_cast<float4*>(p)[2 * i + h], b = reinterpret_cast<float4*>(m)[2 * i + h];
      const float4 c = reinterpret_cast<float4*>(v)[2 * i + h], d = reinterpret_cast<const float4*>(g)[2 * i + h];
      pa[4 * h] = a.x; pa[4 * h + 1] = a.y; pa[4 * h + 2] = a.z; pa[4 * h + 3] = a.w;
      ma[4 * h] = b.x; ma[4 * h + 1] = b.y; ma[4 * h + 2] = b.z; ma[4 * h + 3] = b.w;
      va[4 * h] = c.x; va[4 * h + 1] = c.y; va[4 * h + 2] = c.z; va[4 * h + 3] = c.w;
      ga[4 * h] = d.x; ga[4 * h + 1] = d.y; ga[4 * h + 2] = d.z; ga[4 * h + 3] = d.w;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gr = ga[k] * scale;
      float x = pa[k] * (1.f - lr * wd);
      ma[k] = beta1 * ma[k] + (1.f - beta1) * gr;
      va[k] = beta2 * va[k] + (1.f - beta2) * gr * gr;
      x -= lr * inv_bc1 * ma[k] / (sqrtf(va[k]) * inv_sqrt_bc2 + eps);
      pa[k] = x;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      reinterpret_cast<float4*>(p)[2 * i + h] = make_float4(pa[4 * h], pa[4 * h + 1], pa[4 * h + 2], pa[4 * h + 3]);
      reinterpret_cast<float4*>(m)[2 * i + h] = make_float4(ma[4 * h], ma[4 * h + 1], ma[4 * h + 2], ma[4 * h + 3]);
      reinterpret_cast<float4*>(v)[2 * i + h] = make_float4(va[4 * h], va[4 * h + 1], va[4 * h + 2], va[4 * h + 3]);
    }
    const uint4 packed = make_uint4(pack_bf16(pa[0], pa[1]), pack_bf16(pa[2], pa[3]), pack_bf16(pa[4], pa[5]), pack_bf16(pa[6], pa[7]));
    if (mc_params != nullptr) {
      multimem_st_b32x4(mc_params + lo + i * 8, packed);
    } else {
      for (int r = 0; r < n; ++r) {
        const int dst = (rank + r) % n;
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[dst]) + lo + i * 8) = packed;
      }
    }
  }
  if (ready.p[0] != nullptr) {
    // "parameters of this bucket are ready" to every rank, once the LAST block has stored its part: every
    // thread fences its own (peer / multicast) stores, the block's arrival is counted, and the block that
    // completes the count publishes the new update count with release stores at system scope.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      int* mine = reinterpret_cast<int*>(ready.p[rank]);
      const unsigned int prev = atomicAdd(reinterpret_cast<unsigned int*>(mine + READY_CNT0 + bucket), 1u);
      if (prev == gridDim.x - 1) __threadfence_system();           // acquire side of the count: see every block's stores
      const proto::ReadyLayout layout{READY_STRIDE, READY_EPOCH0, READY_CNT0};
      proto::publish_if_last<DeviceMem>(reinterpret_cast<int* const*>(ready.p), n, rank, bucket, layout, prev, gridDim.x);
    }
  }
}

// One warp: wait until every rank's update of `bucket` has arrived here (see READY_* in common.cuh). Queued at the
// top of a step in front of the first kernels that read parameters no GEMM waits for itself (embedding, norms).
__global__ void wait_params_ready_kernel(const int* ready_local, int bucket, int n, unsigned int* status) {
  wait_params_ready(ready_local, bucket, n, (int)threadIdx.x, status, 46);
}

}  // namespace tlm

using namespace tlm;

static PeerPtrs to_ptrs(void* const* src, int n) {
  PeerPtrs out{};
  for (int i = 0; i < n && i < MAX_PEERS; ++i) out.p[i] = src[i];
  return out;
}

TLM_API int tlm_peer_barrier(void* const* flag_ptrs, int rank, int n, int epoch, cudaStream_t st) {
  if (n > MAX_PEERS) return -6;
  peer_barrier_kernel<<<1, 32, 0, st>>>(to_ptrs(flag_ptrs, n), rank, n, epoch, status_word());
  count_launch();
  return launch_status();
}

// Stream-ordered bounded wait on a device-visible int32 flag (one thread). Work queued behind it starts when
// the flag reaches `expect`, or after `limit_ns` with the timeout recorded in the device status word.
TLM_API int tlm_wait_flag(const int* flag, int expect, unsigned long long limit_ns, cudaStream_t st) {
  if (flag == nullptr || limit_ns == 0 || limit_ns > 10000000000ull) return -6;
  wait_flag_kernel<<<1, 1, 0, st>>>(flag, expect, limit_ns, status_word());
  count_launch();
  return launch_status();
}

TLM_API int tlm_reduce_scatter_blocks() { return 4 * num_sms(); }

// Grid of a reduce-scatter launch: all of it by default; `max_blocks` > 0 caps it (a bucket that is reduced
// while the backward pass still runs should leave the SMs to the GEMMs: a few dozen blocks keep NVLink busy).
static int rs_grid(int max_blocks) {
  const int full = tlm_reduce_scatter_blocks();
  return (max_blocks > 0 && max_blocks < full) ? max_blocks : full;
}

TLM_API int tlm_ready_ints() { return READY_INTS; }
TLM_API int tlm_ready_max_buckets() { return READY_MAX_BUCKETS; }

TLM_API int tlm_wait_params_ready(const int* ready_local, int bucket, int n, cudaStream_t st) {
  if (ready_local == nullptr || bucket < 0 || bucket >= READY_MAX_BUCKETS || n < 1 || n > READY_STRIDE) return -6;
  wait_params_ready_kernel<<<1, 32, 0, st>>>(ready_local, bucket, n, status_word());
  count_launch();
  return launch_status();
}

// partials: >= tlm_reduce_scatter_blocks() floats; sumsq_out: 1 float.
TLM_API int tlm_reduce_scatter(void* const* grad_ptrs, const float* mc_grads, void* const* flag_ptrs, float* out,
                               float* partials, float* sumsq_out, long long lo, long long len, int rank, int n,
                               int epoch, int max_blocks, cudaStream_t st) {
  if (n > MAX_PEERS || len % 4 != 0 || lo % 4 != 0) return -6;
  const int blocks = rs_grid(max_blocks);
  // Under the backward pass (max_blocks > 0) the blocks are small (128 threads, a few thousand registers), so that
  // they fit on an SM next to a resident GEMM block instead of waiting for it or keeping the next one out.
  reduce_scatter_kernel<<<blocks, max_blocks > 0 ? 128 : 512, 0, st>>>(to_ptrs(grad_ptrs, n), mc_grads, to_ptrs(flag_ptrs, n),
                                                                      out, partials, lo, len, rank, n, epoch, status_word());
  sum_partials_kernel<<<1, 256, 0, st>>>(partials, blocks, sumsq_out, to_ptrs(flag_ptrs, n), rank, epoch);
  count_launch(2);
  return launch_status();
}

// bf16 wire: elements [cast_lo, cast_lo + cast_n) of `grads` (this rank's fp32 buffer) are rounded into the same
// elements of `wire_local` (this rank's symmetric bf16 buffer; the range is the bucket every rank is about to
// reduce), then the slice [lo, lo+len) is summed over all ranks' wire buffers into `out` (fp32).
TLM_API int tlm_reduce_scatter_bf16(const float* grads, void* wire_local, long long cast_lo, long long cast_n,
                                    void* const* wire_ptrs, const void* mc_wire, void* const* flag_ptrs, float* out,
                                    float* partials, float* sumsq_out, long long lo, long long len, int rank, int n,
                                    int epoch, int max_blocks, cudaStream_t st) {
  if (n > MAX_PEERS || len % 8 != 0 || lo % 8 != 0 || cast_n % 8 != 0 || cast_lo % 8 != 0) return -6;
  long long cb = (cast_n / 8 + 255) / 256;
  const long long cap = max_blocks > 0 ? max_blocks : 8LL * num_sms();
  if (cb > cap) cb = cap;
  cast_bf16_kernel<<<(int)(cb < 1 ? 1 : cb), 256, 0, st>>>(grads + cast_lo, (__nv_bfloat16*)wire_local + cast_lo, cast_n);
  const int blocks = rs_grid(max_blocks);
  reduce_scatter_bf16_kernel<<<blocks, max_blocks > 0 ? 128 : 512, 0, st>>>(to_ptrs(wire_ptrs, n), (const __nv_bfloat16*)mc_wire, to_ptrs(flag_ptrs, n),
                                                     out, partials, lo, len, rank, n, epoch, status_word());
  sum_partials_kernel<<<1, 256, 0, st>>>(partials, blocks, sumsq_out, to_ptrs(flag_ptrs, n), rank, epoch);
  count_launch(3);
  return launch_status();
}

// `hyper` (optional, device, 3 floats: lr, 1/(1-beta1^t), 1/sqrt(1-beta2^t)) overrides the by-value arguments, so
// that the launch is identical from step to step. `ready_ptrs` (optional: every rank's READY_INTS-word symmetric
// flag array): the kernel ends by publishing "bucket `bucket` updated" to all ranks (see READY_* in common.cuh).
TLM_API int tlm_adamw_gather(float* p, float* m, float* v, const float* g, void* const* param_ptrs, void* mc_params,
                             const float* scale, long long lo, long long len, int rank, int n, float lr, float beta1,
                             float beta2, float eps, float wd, float inv_bc1, float inv_sqrt_bc2, const float* hyper,
                             void* const* ready_ptrs, int bucket, cudaStream_t st) {
  if (n > MAX_PEERS || len % 8 != 0 || lo % 8 != 0) return -6;
  if (ready_ptrs != nullptr && (bucket < 0 || bucket >= READY_MAX_BUCKETS || n > READY_STRIDE)) return -6;
  PeerPtrs ready{};
  if (ready_ptrs != nullptr) ready = to_ptrs(ready_ptrs, n);
  long long blocks = (len / 8 + 255) / 256;
  if (blocks > 8LL * num_sms()) blocks = 8LL * num_sms();
  if (blocks < 1) blocks = 1;
  adamw_gather_kernel<<<(int)blocks, 256, 0, st>>>(p, m, v, g, to_ptrs(param_ptrs, n), (__nv_bfloat16*)mc_params, scale, lo,
                                                   len, rank, n, lr, beta1, beta2, eps, wd, inv_bc1, inv_sqrt_bc2, hyper, ready,
                                                   bucket);
  count_launch();
  return launch_status();
}

// out = scale * sum over ranks of *in (fp32). slots: symmetric array of 2 * 16 floats, flags: symmetric flag array.
TLM_API int tlm_peer_allreduce_scalar(void* const* slot_ptrs, void* const* flag_ptrs, const float* in, float* out, float scale,
                                      int rank, int n, int epoch, cudaStream_t st) {
  if (n > MAX_PEERS) return -6;
  peer_allreduce_scalar_kernel<<<1, 32, 0, st>>>(to_ptrs(slot_ptrs, n), to_ptrs(flag_ptrs, n), in, out, scale, rank, n, epoch,
                                                 status_word());
  count_launch();
  return launch_status();
}
