// Expert-parallel token exchange over NVLink peer memory.
//
// Dispatch and combine are the same primitive: row i of a local bf16 matrix is
// stored into row dest_row[i] of rank dest_rank[i]'s receive buffer (symmetric
// memory). All routing arrays stay on the device, so no split sizes ever travel
// to the host: the sender computes every destination row from the all-ranks
// count table, and the receiver's buffer is already grouped by expert.
//
//   peer_put_i32       : publish a small int32 row (per-expert counts) into every peer's table
//   peer_scatter_rows  : out[dest_rank[i]][dest_row[i], :] = src[src_idx ? src_idx[i] : i, :]
//                        for i < *n_ptr (rows with dest_rank < 0 are skipped)
// Completion is published with the flag barrier of collectives.cu.
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
__global__ void peer_scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, const long long* __restrict__ src_idx,
                                         const int* __restrict__ dest_rank, const long long* __restrict__ dest_row,
                                         RowPeers dst, int D, const long long* __restrict__ n_ptr, long long n_max,
                                         long long dst_rows, unsigned int* status) {
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
    const long long s = src_idx != nullptr ? src_idx[i] : i;
    const uint4* sp = reinterpret_cast<const uint4*>(src + s * D);
    uint4* dp = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[dr]) + row * D);
    for (int v = lane; v < D / 8; v += 32) dp[v] = sp[v];
  }
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

TLM_API int tlm_peer_scatter_rows(const void* src, const long long* src_idx, const int* dest_rank,
                                  const long long* dest_row, void* const* dst_ptrs, int n_peers, int D,
                                  const long long* n_ptr, long long n_max, long long dst_rows, cudaStream_t st) {
  if (n_peers > 16 || D % 8 != 0) return -6;
  if (n_max <= 0) return 0;
  RowPeers d{};
  for (int i = 0; i < n_peers; ++i) d.p[i] = dst_ptrs[i];
  long long blocks = (n_max * 32 + 255) / 256;
  if (blocks > 16LL * num_sms()) blocks = 16LL * num_sms();
  peer_scatter_rows_kernel<<<(int)blocks, 256, 0, st>>>((const __nv_bfloat16*)src, src_idx, dest_rank, dest_row, d, D, n_ptr,
                                                        n_max, dst_rows, status_word());
  count_launch();
  return launch_status();
}
