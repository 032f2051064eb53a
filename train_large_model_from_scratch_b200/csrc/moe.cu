// Mixture-of-experts routing and token exchange.
//
// Routing (all on the device, no sort, no host sync):
//   moe_route    one warp per token: top-k of the raw router logits (ties -> lower expert id), softmax over
//                the k winners, per-block expert histogram
//   moe_scan     block histograms -> exclusive prefix per (block, expert), per-expert totals and bases
//   moe_slot     position of every (token, slot) pair in expert-major / token-minor order (the order a
//                stable sort by expert id would give) and the inverse permutation
//   moe_route_bwd  gradient of softmax-over-top-k scattered into a zero-filled [M, E] logit gradient
// Data movement:
//   moe_gather   out[i, :] = scale[i] * x[order[i] / k, :]               (pairs -> expert-major rows)
//   moe_combine  out[t, :] = sum_s w[t, s] * y[pos[t, s], :]             (expert-major rows -> tokens)
//   moe_pair_dot dw[t, s]  = < d_out[t, :], y[pos[t, s], :] >
//   moe_plan     expert-parallel routing plan from the all-ranks count table (send route, row ranges, back route)
// Expert parallelism over NVLink peer memory (symmetric buffers):
//   peer_put_i32       publish a small int32 row (per-expert counts) into every peer's table
//   peer_scatter_rows  out[dest_rank[i]][dest_row[i], :] = scale[j] * src[j / src_div, :],  j = src_idx ? src_idx[i] : i
//                      for i < *n_ptr (rows with dest_rank < 0 are skipped); dispatch and combine are this
//                      one primitive, the receiver's buffer is already grouped by expert.
// Completion of an exchange is published with the flag barrier of collectives.cu.
#include "common.cuh"

namespace tlm {

struct RowPeers { void* p[16]; };

__global__ void peer_put_i32_kernel(const int* __restrict__ src, int n, RowPeers dst, int n_peers, long long offset) {
  const int total = n * n_peers;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int peer = i / n, k = i - peer * n;
    reinterpret_cast<int*>(dst.p[peer])[offset + k] = src[k];
  }
}

// one warp per row; D multiple of 8
__global__ void peer_scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ src_idx, int src_div,
                                         const float* __restrict__ row_scale, const int* __restrict__ dest_rank,
                                         const long long* __restrict__ dest_row, RowPeers dst, int D,
                                         const long long* __restrict__ n_ptr, long long n_max, long long dst_rows,
                                         unsigned int* status) {
  const int lane = threadIdx.x & 31;
  long long n = n_ptr != nullptr ? *n_ptr : n_max;
  if (n > n_max) n = n_max;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
    const int dr = dest_rank[i];
    if (dr < 0) continue;
    const long long row = dest_row[i];
    if (row < 0 || row >= dst_rows) {                        // never store outside the receive buffer
      if (lane == 0) report_status(status, (60u << 8) | 1u);
      continue;
    }
    const long long s = src_idx != nullptr ? (long long)(src_idx[i] / src_div) : i;
    const uint4* sp = reinterpret_cast<const uint4*>(src + s * D);
    uint4* dp = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[dr]) + row * D);
    if (row_scale == nullptr) {
      for (int v = lane; v < D / 8; v += 32) dp[v] = sp[v];
    } else {
      const float sc = row_scale[src_idx != nullptr ? src_idx[i] : i];
      for (int v = lane; v < D / 8; v += 32) {
        const uint4 a = sp[v];
        const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), a2 = unpack_bf16(a.z), a3 = unpack_bf16(a.w);
        dp[v] = make_uint4(pack_bf16(a0.x * sc, a0.y * sc), pack_bf16(a1.x * sc, a1.y * sc),
                           pack_bf16(a2.x * sc, a2.y * sc), pack_bf16(a3.x * sc, a3.y * sc));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- routing
constexpr int ROUTE_TOKENS = 128;      // tokens per block (route and slot kernels use the same split)
constexpr int ROUTE_MAX_E = 256, ROUTE_MAX_K = 8;

// logits [M, E] bf16 (row pitch ld). weights [M, k] fp32, experts [M, k] int32, block_hist [blocks, E].
__global__ void __launch_bounds__(256)
moe_route_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, int M, int E, int k,
                 float* __restrict__ weights, int* __restrict__ experts, int* __restrict__ block_hist) {
  __shared__ int hist[ROUTE_MAX_E];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t_end = min(M, (int)(blockIdx.x + 1) * ROUTE_TOKENS);
  for (int t = blockIdx.x * ROUTE_TOKENS + warp; t < t_end; t += warps) {
    float v[ROUTE_MAX_E / 32];
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_E / 32; ++i) {
      const int e = lane + 32 * i;
      v[i] = e < E ? __bfloat162float(logits[(long long)t * ld + e]) : -INFINITY;
    }
    float top_v[ROUTE_MAX_K];
    int top_e[ROUTE_MAX_K];
    for (int s = 0; s < k; ++s) {
      float bv = -INFINITY; int be = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < ROUTE_MAX_E / 32; ++i) {
        const int e = lane + 32 * i;
        if (e < E && (v[i] > bv || (v[i] == bv && e < be))) { bv = v[i]; be = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oe = __shfl_xor_sync(0xffffffffu, be, o);
        if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
      }
      top_v[s] = bv; top_e[s] = be;
#pragma unroll
      for (int i = 0; i < ROUTE_MAX_E / 32; ++i) if (lane + 32 * i == be) v[i] = -INFINITY;   // taken
    }
    if (lane == 0) {
      float sum = 0.f;
      const float vmax = top_v[0];
      for (int s = 0; s < k; ++s) { top_v[s] = __expf(top_v[s] - vmax); sum += top_v[s]; }
      const float inv = 1.f / sum;
      for (int s = 0; s < k; ++s) {
        weights[(long long)t * k + s] = top_v[s] * inv;
        experts[(long long)t * k + s] = top_e[s];
        atomicAdd(&hist[top_e[s]], 1);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) block_hist[(long long)blockIdx.x * E + e] = hist[e];
}

// In place: block_hist[b][e] -> number of pairs of expert e in blocks < b. counts[e] = total,
// base[e] = sum of counts of experts < e, base[E] = all pairs. One block, thread e owns expert e.
__global__ void moe_scan_kernel(int* __restrict__ block_hist, int n_blocks, int E, int* __restrict__ counts,
                                int* __restrict__ base) {
  __shared__ int tot[ROUTE_MAX_E];
  const int e = threadIdx.x;
  if (e < E) {
    int run = 0;
    for (int b = 0; b < n_blocks; ++b) {
      const int c = block_hist[(long long)b * E + e];
      block_hist[(long long)b * E + e] = run;
      run += c;
    }
    tot[e] = run;
    counts[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < E; ++i) { base[i] = run; run += tot[i]; }
    base[E] = run;
  }
}

// pos[t*k + s] = base[e] + block_off[b][e] + (tokens of this block before t that chose e);  order[pos] = t*k + s.
__global__ void __launch_bounds__(256)
moe_slot_kernel(const int* __restrict__ experts, int M, int E, int k, const int* __restrict__ block_off,
                const int* __restrict__ base, int* __restrict__ pos, int* __restrict__ order) {
  __shared__ int ex[ROUTE_TOKENS * ROUTE_MAX_K];
  const int t0 = blockIdx.x * ROUTE_TOKENS;
  const int nt = min(ROUTE_TOKENS, M - t0);
  for (int i = threadIdx.x; i < nt * k; i += blockDim.x) ex[i] = experts[(long long)t0 * k + i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int e = warp; e < E; e += warps) {
    int run = base[e] + block_off[(long long)blockIdx.x * E + e];
    for (int c = 0; c < nt; c += 32) {
      const int t = c + lane;
      int slot = -1;
      if (t < nt)
        for (int s = 0; s < k; ++s) if (ex[t * k + s] == e) slot = s;
      const unsigned m = __ballot_sync(0xffffffffu, slot >= 0);
      if (slot >= 0) {
        const int p = run + __popc(m & ((1u << lane) - 1u));
        const int pair = (t0 + t) * k + slot;
        pos[pair] = p;
        order[p] = pair;
      }
      run += __popc(m);
    }
  }
}

// d_logits[t, e_s] = w_s * (dw_s - sum_j w_j dw_j); the tensor is zero-filled by the caller.
__global__ void moe_route_bwd_kernel(const float* __restrict__ dw, const float* __restrict__ w, const int* __restrict__ experts,
                                     __nv_bfloat16* __restrict__ d_logits, long long ld, int M, int k) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= M) return;
  float dot = 0.f;
  for (int s = 0; s < k; ++s) dot += w[(long long)t * k + s] * dw[(long long)t * k + s];
  for (int s = 0; s < k; ++s)
    d_logits[(long long)t * ld + experts[(long long)t * k + s]] =
        __float2bfloat16(w[(long long)t * k + s] * (dw[(long long)t * k + s] - dot));
}

// ---------------------------------------------------------------------------------------------- local data movement
// out[i, :] = scale[i] * x[order[i] / k, :]   one warp per row
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ order, int k,
                                  const float* __restrict__ scale, __nv_bfloat16* __restrict__ out, long long P, int D) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < P; i += warps) {
    const long long srow = order[i] / k;
    const uint4* sp = reinterpret_cast<const uint4*>(x + srow * D);
    uint4* dp = reinterpret_cast<uint4*>(out + i * D);
    if (scale == nullptr) {
      for (int v = lane; v < D / 8; v += 32) dp[v] = sp[v];
    } else {
      const float sc = scale[order[i]];
      for (int v = lane; v < D / 8; v += 32) {
        const uint4 a = sp[v];
        const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), a2 = unpack_bf16(a.z), a3 = unpack_bf16(a.w);
        dp[v] = make_uint4(pack_bf16(a0.x * sc, a0.y * sc), pack_bf16(a1.x * sc, a1.y * sc),
                           pack_bf16(a2.x * sc, a2.y * sc), pack_bf16(a3.x * sc, a3.y * sc));
      }
    }
  }
}

// out[t, :] = sum_s w[t*k+s] * y[pos[t*k+s], :]   (w == nullptr: plain sum). One warp per token.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int M, int D, int k) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long t = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < M; t += warps) {
    for (int v = lane; v < D / 8; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < k; ++s) {
        const int p = pos[t * k + s];
        if (p < 0) continue;
        const float ws = w != nullptr ? w[t * k + s] : 1.f;
        const uint4 a = reinterpret_cast<const uint4*>(y + (long long)p * D)[v];
        const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), a2 = unpack_bf16(a.z), a3 = unpack_bf16(a.w);
        acc[0] = fmaf(ws, a0.x, acc[0]); acc[1] = fmaf(ws, a0.y, acc[1]); acc[2] = fmaf(ws, a1.x, acc[2]); acc[3] = fmaf(ws, a1.y, acc[3]);
        acc[4] = fmaf(ws, a2.x, acc[4]); acc[5] = fmaf(ws, a2.y, acc[5]); acc[6] = fmaf(ws, a3.x, acc[6]); acc[7] = fmaf(ws, a3.y, acc[7]);
      }
      reinterpret_cast<uint4*>(out + t * D)[v] =
          make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
    }
  }
}

// dw[pair] = < d_out[pair / k, :], y[pos[pair], :] >   one warp per pair
__global__ void moe_pair_dot_kernel(const __nv_bfloat16* __restrict__ d_out, const __nv_bfloat16* __restrict__ y,
                                    const int* __restrict__ pos, float* __restrict__ dw, long long P, int D, int k) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < P; i += warps) {
    const int p = pos[i];
    float acc = 0.f;
    if (p >= 0) {
      const uint4* a = reinterpret_cast<const uint4*>(d_out + (i / k) * D);
      const uint4* b = reinterpret_cast<const uint4*>(y + (long long)p * D);
      for (int v = lane; v < D / 8; v += 32) {
        const uint4 x = a[v], z = b[v];
        const float2 x0 = unpack_bf16(x.x), x1 = unpack_bf16(x.y), x2 = unpack_bf16(x.z), x3 = unpack_bf16(x.w);
        const float2 z0 = unpack_bf16(z.x), z1 = unpack_bf16(z.y), z2 = unpack_bf16(z.z), z3 = unpack_bf16(z.w);
        acc += x0.x * z0.x + x0.y * z0.y + x1.x * z1.x + x1.y * z1.y + x2.x * z2.x + x2.y * z2.y + x3.x * z3.x + x3.y * z3.y;
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[i] = acc;
  }
}

// ---------------------------------------------------------------------------------------------- expert-parallel plan
// From the all-ranks count table C[src][expert] (ep x E, every rank holds the same copy) derive both routes of
// the token exchange, with no host involvement:
//   receive buffers are laid out expert-major / source-minor, so
//     first row of expert e on its owner      base_g[e]  = sum of tot[e'] over the owner's experts e' < e
//     first row of source s inside expert e   + sum_{s' < s} C[s'][e]
//   send route  (i < P, my sorted pairs)      send_rank[i] = e / E_l,  send_row[i] = that + (i - my_start[e])
//   my experts' row ranges                    row_start[0..E_l], n_recv = row_start[E_l]
//   back route  (r < R, rows I received)      back_rank[r] = source s (or -1 past n_recv),
//                                             back_row[r]  = (first sorted pair of e on s) + offset inside the block
constexpr int PLAN_MAX_EP = 8;

__global__ void __launch_bounds__(256)
moe_plan_kernel(const int* __restrict__ C, int ep, int E, int me, const int* __restrict__ experts, const int* __restrict__ order,
                const int* __restrict__ my_start, int P, long long R, int* __restrict__ send_rank,
                long long* __restrict__ send_row, int* __restrict__ row_start, long long* __restrict__ n_recv,
                int* __restrict__ back_rank, long long* __restrict__ back_row) {
  __shared__ int Cs[PLAN_MAX_EP * ROUTE_MAX_E];
  __shared__ int tot[ROUTE_MAX_E], base_g[ROUTE_MAX_E], pre_me[ROUTE_MAX_E];
  __shared__ int blk_start[ROUTE_MAX_E], blk_cnt[ROUTE_MAX_E], blk_src_start[ROUTE_MAX_E];   // E_l * ep <= E entries
  __shared__ int n_recv_s;
  const int E_l = E / ep, tid = threadIdx.x;
  for (int i = tid; i < ep * E; i += blockDim.x) Cs[i] = C[i];
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    int t = 0, pm = 0;
    for (int s2 = 0; s2 < ep; ++s2) { if (s2 == me) pm = t; t += Cs[s2 * E + e]; }
    tot[e] = t; pre_me[e] = pm;
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    int b = 0;
    for (int e2 = (e / E_l) * E_l; e2 < e; ++e2) b += tot[e2];
    base_g[e] = b;
  }
  __syncthreads();
  for (int b = tid; b < E_l * ep; b += blockDim.x) {         // block b = (local expert, source), expert-major
    const int el = b / ep, s2 = b - el * ep, e = me * E_l + el;
    int st = base_g[e];
    for (int s3 = 0; s3 < s2; ++s3) st += Cs[s3 * E + e];
    int on_src = 0;
    for (int e2 = 0; e2 < e; ++e2) on_src += Cs[s2 * E + e2];
    blk_start[b] = st; blk_cnt[b] = Cs[s2 * E + e]; blk_src_start[b] = on_src;
  }
  if (tid == 0) {
    int n = 0;
    for (int el = 0; el < E_l; ++el) n += tot[me * E_l + el];
    n_recv_s = n;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int el = tid; el <= E_l; el += blockDim.x) row_start[el] = el < E_l ? base_g[me * E_l + el] : n_recv_s;
    if (tid == 0) *n_recv = n_recv_s;
  }
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + tid; i < P; i += stride) {
    const int e = experts[order[i]];
    send_rank[i] = e / E_l;
    send_row[i] = (long long)base_g[e] + pre_me[e] + (i - my_start[e]);
  }
  const int nb = E_l * ep;
  for (long long r = (long long)blockIdx.x * blockDim.x + tid; r < R; r += stride) {
    if (r >= n_recv_s) { back_rank[r] = -1; back_row[r] = 0; continue; }
    // last block with blk_start <= r among non-empty blocks: blocks are contiguous and ascending, so search the ends
    int lo = 0, hi = nb - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if ((long long)blk_start[mid] + blk_cnt[mid] > r) hi = mid; else lo = mid + 1;
    }
    back_rank[r] = lo % ep;
    back_row[r] = (long long)blk_src_start[lo] + (r - blk_start[lo]);
  }
}

static int row_blocks(long long rows) {
  long long blocks = (rows * 32 + 255) / 256;
  if (blocks > 16LL * num_sms()) blocks = 16LL * num_sms();
  return blocks < 1 ? 1 : (int)blocks;
}

}  // namespace tlm

using namespace tlm;

TLM_API int tlm_peer_put_i32(const int* src, int n, void* const* dst_ptrs, int n_peers, long long offset,
                             cudaStream_t st) {
  if (n_peers > 16) return -6;
  RowPeers d{};
  for (int i = 0; i < n_peers; ++i) d.p[i] = dst_ptrs[i];
  peer_put_i32_kernel<<<1, 256, 0, st>>>(src, n, d, n_peers, offset);
  count_launch();
  return launch_status();
}

TLM_API int tlm_peer_scatter_rows(const void* src, const int* src_idx, int src_div, const float* row_scale,
                                  const int* dest_rank, const long long* dest_row, void* const* dst_ptrs, int n_peers,
                                  int D, const long long* n_ptr, long long n_max, long long dst_rows, cudaStream_t st) {
  if (n_peers > 16 || D % 8 != 0 || (src_idx != nullptr && src_div < 1)) return -6;
  if (n_max <= 0) return 0;
  RowPeers d{};
  for (int i = 0; i < n_peers; ++i) d.p[i] = dst_ptrs[i];
  peer_scatter_rows_kernel<<<row_blocks(n_max), 256, 0, st>>>((const __nv_bfloat16*)src, src_idx, src_div, row_scale, dest_rank,
                                                              dest_row, d, D, n_ptr, n_max, dst_rows, status_word());
  count_launch();
  return launch_status();
}

TLM_API int tlm_moe_route_blocks(int M) { return (M + ROUTE_TOKENS - 1) / ROUTE_TOKENS; }

// Routing of M tokens over E experts (E <= 256, k <= 8). Outputs: weights [M,k] fp32, experts [M,k] int32,
// counts [E], base [E+1], pos [M*k], order [M*k] (int32); scratch: block_hist [tlm_moe_route_blocks(M) * E] int32.
TLM_API int tlm_moe_route(const void* logits, long long ld, int M, int E, int k, float* weights, int* experts,
                          int* block_hist, int* counts, int* base, int* pos, int* order, cudaStream_t st) {
  if (E < 1 || E > ROUTE_MAX_E || k < 1 || k > ROUTE_MAX_K || k > E) return -6;
  if (M <= 0) return 0;
  const int blocks = tlm_moe_route_blocks(M);
  moe_route_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)logits, ld, M, E, k, weights, experts, block_hist);
  moe_scan_kernel<<<1, ROUTE_MAX_E, 0, st>>>(block_hist, blocks, E, counts, base);
  moe_slot_kernel<<<blocks, 256, 0, st>>>(experts, M, E, k, block_hist, base, pos, order);
  count_launch(3);
  return launch_status();
}

// Expert-parallel routing plan (see moe_plan_kernel). C: [ep, E] int32 counts of every rank; experts / order /
// my_start: this rank's routing (`tlm_moe_route` outputs experts, order, base). Outputs: send_rank [P] int32,
// send_row [P] int64, row_start [E/ep + 1] int32, n_recv [1] int64, back_rank [R] int32, back_row [R] int64.
TLM_API int tlm_moe_plan(const int* C, int ep, int E, int me, const int* experts, const int* order, const int* my_start,
                         int P, long long R, int* send_rank, long long* send_row, int* row_start, long long* n_recv,
                         int* back_rank, long long* back_row, cudaStream_t st) {
  if (ep < 1 || ep > PLAN_MAX_EP || E < ep || E > ROUTE_MAX_E || E % ep != 0 || me < 0 || me >= ep) return -6;
  long long n = P > R ? P : R;
  long long blocks = (n + 255) / 256;
  if (blocks > 2LL * num_sms()) blocks = 2LL * num_sms();
  if (blocks < 1) blocks = 1;
  moe_plan_kernel<<<(int)blocks, 256, 0, st>>>(C, ep, E, me, experts, order, my_start, P, R, send_rank, send_row, row_start,
                                               n_recv, back_rank, back_row);
  count_launch();
  return launch_status();
}

TLM_API int tlm_moe_route_bwd(const float* dw, const float* w, const int* experts, void* d_logits, long long ld, int M,
                              int k, cudaStream_t st) {
  if (M <= 0) return 0;
  moe_route_bwd_kernel<<<(M + 255) / 256, 256, 0, st>>>(dw, w, experts, (__nv_bfloat16*)d_logits, ld, M, k);
  count_launch();
  return launch_status();
}

TLM_API int tlm_moe_gather(const void* x, const int* order, int k, const float* scale, void* out, long long P, int D,
                           cudaStream_t st) {
  if (D % 8 != 0) return -6;
  if (P <= 0) return 0;
  moe_gather_kernel<<<row_blocks(P), 256, 0, st>>>((const __nv_bfloat16*)x, order, k, scale, (__nv_bfloat16*)out, P, D);
  count_launch();
  return launch_status();
}

TLM_API int tlm_moe_combine(const void* y, const int* pos, const float* w, void* out, int M, int D, int k,
                            cudaStream_t st) {
  if (D % 8 != 0) return -6;
  if (M <= 0) return 0;
  moe_combine_kernel<<<row_blocks(M), 256, 0, st>>>((const __nv_bfloat16*)y, pos, w, (__nv_bfloat16*)out, M, D, k);
  count_launch();
  return launch_status();
}

TLM_API int tlm_moe_pair_dot(const void* d_out, const void* y, const int* pos, float* dw, long long P, int D, int k,
                             cudaStream_t st) {
  if (D % 8 != 0) return -6;
  if (P <= 0) return 0;
  moe_pair_dot_kernel<<<row_blocks(P), 256, 0, st>>>((const __nv_bfloat16*)d_out, (const __nv_bfloat16*)y, pos, dw, P, D, k);
  count_launch();
  return launch_status();
}
