// Causal GQA flash attention, backward, on tcgen05 / TMEM.
//
// Inputs: packed qkv[B,T,Hq+2Hkv,hd], o[B,T,Hq,hd], do[B,T,Hq,hd] (bf16),
// lse[B,Hq,T] (fp32). Output: dqkv[B,T,Hq+2Hkv,hd] (bf16) in the packed layout,
// so the QKV projection's dgrad/wgrad GEMMs consume one tensor.
//
// Three launches:
//   1. delta[b,h,t] = sum_d do*o
//   2. main kernel: one CTA per (128-row KV tile, batch, KV head). K and V stay in
//      shared memory; the CTA walks over every query head of the group and every
//      query tile at or below the diagonal. Per step five MMAs run on the
//      tensor cores:   S = Q K^T,  dP = dO V^T            (TMEM, fp32)
//                      dV += P^T dO,  dK += dS^T Q         (TMEM accumulators)
//                      dQ  = dS K                          (TMEM, flushed per step)
//      P and dS are written once to shared memory as [q][kv] bf16 tiles in the
//      swizzled operand layout; read as K-major they feed dQ, read as MN-major
//      they are P^T / dS^T, and Q / dO / K / V tiles are used as loaded (MN-major
//      where the product needs their transpose), so nothing is transposed.
//      Two softmax warpgroups (one thread per query row, half of the KV columns
//      each) turn S, dP into P, dS; dQ tiles are added to an fp32 buffer with
//      TMA reduce-add tile stores because several KV tiles contribute to one query row.
//      For hd = 64 the next step's S / dP MMAs are issued while the softmax
//      warps still work on the current step.
//   3. dq (fp32, [B,Hq,T,hd]) -> bf16 into dqkv; with RoPE tables this pass also applies the transposed rotation to
//      dQ (from the fp32 accumulator) and to the dK slots the main kernel wrote, so the packed gradient that leaves
//      is the gradient of the UN-rotated q and k and no separate RoPE pass runs.
// A second instantiation of the main kernel (SCATTER) serves Ulysses sequence parallelism: its dK / dV epilogue
// rotates dK itself and stores the rows straight into the sequence owners' packed gradient buffers, and the
// conversion pass does the same for dQ. The plain instantiation carries none of that code: this kernel's main loop
// is sensitive to anything that changes its register allocation, and in-step timing (not the isolated kernel
// benchmark) decides what stays in it.
// Every wait is bounded; on a timeout the CTA records a status code, leaves its
// loops and still releases its tensor memory.
#include "common.cuh"

namespace tlm {

constexpr int AB_TILE = 128, AB_THREADS = 320, AB_MAX_DST = 8;

struct AttnBwdDst {
  __nv_bfloat16* p[AB_MAX_DST];
  int n, rows, heads;
};

struct AttnBwdParams {
  __nv_bfloat16* dqkv;
  float* dq_acc;            // [B,Hq,T,hd] fp32, zeroed by the launcher
  const float* lse;
  const float* delta;
  int B, T, Hq, Hkv;
  float scale, scale_log2;
  unsigned int* status;
  int hd;                   // head dim in memory; 32 runs on the HD = 64 kernel with zero-filled upper columns
  // Transposed RoPE on the way out (tables cos / sin [T, hd], fp32, row = position; nullptr: off):
  //   dx[j] = dy[j] c[j] + dy[j+h] s[j+h],  dx[j+h] = dy[j+h] c[j+h] - dy[j] s[j]   (h = hd / 2).
  const float* cosT;
  const float* sinT;
  // SCATTER instantiation only: head -> sequence return of the packed gradient (Ulysses backward). Row t of local
  // head slot s is stored into
  //   dst[t / dst_rows][b, t % dst_rows, head(s), :]     (bf16 [B, dst_rows, dst_heads, hd] per rank)
  // with head(s) = dst_q0 + s for q slots, dst_k0 + s for k, dst_v0 + s for v (peer-mapped addresses, plain
  // 16-byte stores).
  __nv_bfloat16* dst[AB_MAX_DST];
  int n_dst, dst_rows, dst_heads, dst_q0, dst_k0, dst_v0;
  int head_group;          // (batch, KV head) pairs per group of the heavy-first block order (see heavy_first_decode)
};

template <int HD>
struct AttnBwdCfg {
  // Q / dO ring. Three stages for hd 64: the MMA warp issues S / dP of step it+1 before dV / dK / dQ of step
  // it, so the load of step it+1 must have been started a whole step earlier (when step it-2 retired) for its
  // latency to stay off the tensor pipe's critical path.
  static constexpr int STAGES = HD == 64 ? 3 : 1;
  static constexpr bool PIPELINED = HD == 64;            // dQ has its own TMEM columns
  static constexpr int TILE_BYTES = AB_TILE * HD * 2;
  static constexpr int PD_BYTES = AB_TILE * AB_TILE * 2;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + TILE_BYTES;
  static constexpr int OFF_Q = OFF_V + TILE_BYTES;
  static constexpr int OFF_DO = OFF_Q + STAGES * TILE_BYTES;
  static constexpr int OFF_P = OFF_DO + STAGES * TILE_BYTES;
  static constexpr int OFF_DS = OFF_P + PD_BYTES;
  static constexpr int OFF_DQS = OFF_DS + PD_BYTES;      // dQ staging: one [32 rows][32 fp32] swizzled box per softmax warp
  static constexpr int DQS_BYTES = 8 * 4096;
  static constexpr int OFF_BAR = OFF_DQS + DQS_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
  static constexpr uint32_t S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 256 + HD;
  // hd 64: dQ has two 64-column buffers (steps alternate), so dQ of step it can be issued while the softmax
  // warps still drain dQ of step it-1. hd 128: dQ reuses the S columns (no spare tensor memory).
  static constexpr uint32_t DQ_COL = HD == 64 ? 384 : 0;
  static constexpr uint32_t DQ_BUF_COLS = HD == 64 ? 64 : 0;
};

// delta[b, h, t] = sum_c o[b, t, h, c] * dout[b, t, h, c]. One block per (b, 32 consecutive t): that slab of o
// and dout is contiguous, hd / 8 lanes share a row with 16-byte loads (four rows in flight per lane), the row sums
// are staged in shared memory so that the [B, Hq, T] output is written as whole 128-byte lines.
constexpr int DELTA_T = 32, DELTA_THREADS = 256;

__global__ void __launch_bounds__(DELTA_THREADS)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                  float* __restrict__ delta, int B, int T, int Hq, int hd) {
  extern __shared__ float delta_s[];                       // [Hq][DELTA_T + 1]
  const int tiles_t = (T + DELTA_T - 1) / DELTA_T;
  const int b = blockIdx.x / tiles_t, t0 = (blockIdx.x % tiles_t) * DELTA_T;
  const int nt = min(DELTA_T, T - t0);
  const int lpr = hd >> 3;                                 // lanes per row: 4, 8 or 16
  const int sub = threadIdx.x % lpr, slot = threadIdx.x / lpr, slots = DELTA_THREADS / lpr;
  const int rows = nt * Hq;                                // row rr = tl * Hq + h
  const long long base = ((long long)b * T + t0) * Hq * hd;
  const uint4* op = reinterpret_cast<const uint4*>(o + base) + sub;
  const uint4* dp = reinterpret_cast<const uint4*>(dout + base) + sub;
  for (int rb = 0; rb < rows; rb += 4 * slots) {          // trip count is uniform: the shuffles below need whole warps
    const int r0 = rb + slot;
    uint4 a[4], d[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int rr = r0 + u * slots;
      if (rr < rows) { a[u] = op[(long long)rr * lpr]; d[u] = dp[(long long)rr * lpr]; }
      else { a[u] = make_uint4(0, 0, 0, 0); d[u] = a[u]; }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, dw[4] = {d[u].x, d[u].y, d[u].z, d[u].w};
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 x = unpack_bf16(aw[k]), y = unpack_bf16(dw[k]);
        acc = fmaf(x.x, y.x, fmaf(x.y, y.y, acc));
      }
      for (int off = lpr >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      const int rr = r0 + u * slots;
      if (sub == 0 && rr < rows) delta_s[(rr % Hq) * (DELTA_T + 1) + rr / Hq] = acc;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < Hq * DELTA_T; i += DELTA_THREADS) {
    const int h = i / DELTA_T, tl = i % DELTA_T;
    if (tl < nt) delta[((long long)b * Hq + h) * T + t0 + tl] = delta_s[h * (DELTA_T + 1) + tl];
  }
}

// dq_acc (fp32 [B, Hq, T, hd]) * scale -> bf16 q-head slots of dqkv, 8 low columns and their 8 partner columns
// (j + hd / 2) per thread so that the transposed rotation (see AttnBwdParams) can be applied on the way.
// `rot_k` (only without a head -> sequence return): the Hkv k-head slots of dqkv, written as bf16 by the main kernel, are
// rotated in place by further work items (heads Hq .. Hq + Hkv - 1).
__global__ void attn_dq_convert_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, int B, int T,
                                       int Hq, int heads_total, int hd, float scale, const float* __restrict__ cosT,
                                       const float* __restrict__ sinT, const AttnBwdDst d, int dst_q0, int rot_k) {
  const int half = hd / 2, vec = half / 8;
  const int heads = Hq + rot_k;
  const long long total = (long long)B * heads * T * vec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % vec) * 8;
    long long r = i / vec;
    const int t = (int)(r % T); r /= T;
    const int h = (int)(r % heads); const long long b = r / heads;
    float lo[8], hi[8];
    if (h < Hq) {
      const float* src = dq_acc + (((long long)b * Hq + h) * T + t) * hd + j;
      *reinterpret_cast<float4*>(lo) = *reinterpret_cast<const float4*>(src);
      *reinterpret_cast<float4*>(lo + 4) = *reinterpret_cast<const float4*>(src + 4);
      *reinterpret_cast<float4*>(hi) = *reinterpret_cast<const float4*>(src + half);
      *reinterpret_cast<float4*>(hi + 4) = *reinterpret_cast<const float4*>(src + half + 4);
#pragma unroll
      for (int k = 0; k < 8; ++k) { lo[k] *= scale; hi[k] *= scale; }
    } else {                                             // a k head: bf16 in, rotated bf16 out, same place
      const __nv_bfloat16* src = dqkv + ((b * T + t) * heads_total + h) * (long long)hd + j;
      const uint4 a = *reinterpret_cast<const uint4*>(src), c = *reinterpret_cast<const uint4*>(src + half);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 x = unpack_bf16(aw[k]), y = unpack_bf16(cw[k]);
        lo[2 * k] = x.x; lo[2 * k + 1] = x.y; hi[2 * k] = y.x; hi[2 * k + 1] = y.y;
      }
    }
    if (cosT != nullptr) {
      const float* c = cosT + (long long)t * hd + j;
      const float* sn = sinT + (long long)t * hd + j;
      float cl[8], ch[8], sl[8], sh[8];
      *reinterpret_cast<float4*>(cl) = *reinterpret_cast<const float4*>(c);
      *reinterpret_cast<float4*>(cl + 4) = *reinterpret_cast<const float4*>(c + 4);
      *reinterpret_cast<float4*>(ch) = *reinterpret_cast<const float4*>(c + half);
      *reinterpret_cast<float4*>(ch + 4) = *reinterpret_cast<const float4*>(c + half + 4);
      *reinterpret_cast<float4*>(sl) = *reinterpret_cast<const float4*>(sn);
      *reinterpret_cast<float4*>(sl + 4) = *reinterpret_cast<const float4*>(sn + 4);
      *reinterpret_cast<float4*>(sh) = *reinterpret_cast<const float4*>(sn + half);
      *reinterpret_cast<float4*>(sh + 4) = *reinterpret_cast<const float4*>(sn + half + 4);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float a = lo[k], bb = hi[k];
        lo[k] = a * cl[k] + bb * sh[k];
        hi[k] = bb * ch[k] - a * sl[k];
      }
    }
    __nv_bfloat16* dst;
    if (d.n > 0) {
      const int owner = t / d.rows, tl = t - owner * d.rows;
      if (owner >= d.n) continue;
      dst = d.p[owner] + ((b * d.rows + tl) * d.heads + dst_q0 + h) * (long long)hd + j;
    } else {
      dst = dqkv + ((b * T + t) * heads_total + h) * (long long)hd + j;
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]), pack_bf16(lo[4], lo[5]), pack_bf16(lo[6], lo[7]));
    *reinterpret_cast<uint4*>(dst + half) = make_uint4(pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]), pack_bf16(hi[4], hi[5]), pack_bf16(hi[6], hi[7]));
  }
}

template <int HD, bool SCATTER>
__global__ void __launch_bounds__(AB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_dq, const AttnBwdParams p) {
  using C = AttnBwdCfg<HD>;
  constexpr int KB = HD / 64;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sal = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t bar0 = sbase + C::OFF_BAR;
  // barriers: 0,1 dq_consumed[buffer] (hd 64)  4 kv_full  5 sdp_full  6 sdp_consumed  7 pds_full  8 dq_full
  //           9 dq_consumed (hd 128)  10.. qdo_full[stage]  13.. qdo_empty[stage]
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sal + C::OFF_BAR + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (p.T + AB_TILE - 1) / AB_TILE;
  int j, bh;                                                  // KV tile (tile 0 has the most query tiles), (batch, KV head)
  heavy_first_decode((int)blockIdx.x, n_tiles, p.B * p.Hkv, p.head_group, j, bh);
  const int b = bh / p.Hkv, kvh = bh % p.Hkv;
  const int rep = p.Hq / p.Hkv;
  const int per_head = n_tiles - j;                           // query tiles j..n_tiles-1
  const int n_it = rep * per_head;
  const int heads_total = p.Hq + 2 * p.Hkv;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 16; ++i) mbar_init(bar(i), (i == 0 || i == 1 || i == 6 || i == 7 || i == 9) ? 8 : 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_qkv);
    tma_prefetch_desc(&tm_do);
    tma_prefetch_desc(&tm_dq);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(bar(4), 2 * C::TILE_BYTES);
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) {
        tma_load_4d(sbase + C::OFF_K + kb * 16384, &tm_qkv, bar(4), kb * 64, p.Hq + kvh, j * AB_TILE, b);
        tma_load_4d(sbase + C::OFF_V + kb * 16384, &tm_qkv, bar(4), kb * 64, p.Hq + p.Hkv + kvh, j * AB_TILE, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it % C::STAGES;
        const uint32_t ph = (uint32_t)(it / C::STAGES) & 1u;
        if (!mbar_wait(bar(13 + st), ph ^ 1u, 21, abort_flag, p.status)) break;
        const int hq = kvh * rep + it / per_head, qi = j + it % per_head;
        mbar_expect_tx(bar(10 + st), 2 * C::TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
          tma_load_4d(sbase + C::OFF_Q + st * C::TILE_BYTES + kb * 16384, &tm_qkv, bar(10 + st), kb * 64, hq, qi * AB_TILE, b);
          tma_load_4d(sbase + C::OFF_DO + st * C::TILE_BYTES + kb * 16384, &tm_do, bar(10 + st), kb * 64, hq, qi * AB_TILE, b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(AB_TILE, AB_TILE, 0, 0);     // S, dP : A, B K-major
      constexpr uint32_t idesc_t = umma_idesc_bf16(AB_TILE, HD, 1, 1);          // dV, dK: A, B MN-major
      constexpr uint32_t idesc_q = umma_idesc_bf16(AB_TILE, HD, 0, 1);          // dQ    : A K-major, B MN-major
      const uint32_t sk = sbase + C::OFF_K, sv = sbase + C::OFF_V, sp = sbase + C::OFF_P, sds = sbase + C::OFF_DS;
      // descriptors of the resident K / V tiles and of the P / dS tiles, built once
      const uint64_t dk_k = umma_smem_desc(sk, 16, 1024), dv_k = umma_smem_desc(sv, 16, 1024);     // K-major views
      const uint64_t dk_mn = umma_smem_desc(sk, 16384, 1024);                                      // K as MN-major B (dQ)
      const uint64_t dp_mn = umma_smem_desc(sp, 16384, 1024), dds_mn = umma_smem_desc(sds, 16384, 1024);
      const uint64_t dds_k = umma_smem_desc(sds, 16, 1024);
      auto issue_s_dp = [&](int it) -> bool {
        const int st = it % C::STAGES;
        if (!mbar_wait(bar(10 + st), (uint32_t)(it / C::STAGES) & 1u, 22, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint64_t dq_k = umma_smem_desc(sbase + C::OFF_Q + st * C::TILE_BYTES, 16, 1024);
        const uint64_t ddo_k = umma_smem_desc(sbase + C::OFF_DO + st * C::TILE_BYTES, 16, 1024);
#pragma unroll
        for (int t = 0; t < HD / 16; ++t) {
          const uint32_t off = (t >> 2) * 16384 + (t & 3) * 32;
          if (t == 0) umma_bf16(tmem + C::S_COL, dq_k, dk_k, idesc_s, 0);
          else umma_bf16_acc(tmem + C::S_COL, umma_desc_advance(dq_k, off), umma_desc_advance(dk_k, off), idesc_s);
        }
#pragma unroll
        for (int t = 0; t < HD / 16; ++t) {
          const uint32_t off = (t >> 2) * 16384 + (t & 3) * 32;
          if (t == 0) umma_bf16(tmem + C::DP_COL, ddo_k, dv_k, idesc_s, 0);
          else umma_bf16_acc(tmem + C::DP_COL, umma_desc_advance(ddo_k, off), umma_desc_advance(dv_k, off), idesc_s);
        }
        umma_commit(bar(5));
        return true;
      };
      bool ok = mbar_wait(bar(4), 0, 23, abort_flag, p.status);
      if (ok && C::PIPELINED) ok = issue_s_dp(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % C::STAGES;
        const uint32_t par = (uint32_t)it & 1u;
        if (C::PIPELINED) {
          if (it + 1 < n_it) {
            if (!mbar_wait(bar(6), par, 24, abort_flag, p.status)) break;          // S, dP of `it` are in registers
            if (!issue_s_dp(it + 1)) break;
          }
        } else {
          if (it > 0 && !mbar_wait(bar(9), par ^ 1u, 25, abort_flag, p.status)) break;   // dQ(it-1) read out of the S columns
          if (!issue_s_dp(it)) break;
        }
        if (!mbar_wait(bar(7), par, 26, abort_flag, p.status)) break;              // P, dS published
        // this step's dQ buffer was last used by step it-2: its flush is phase (it>>1)-1 of that buffer's barrier
        if (C::PIPELINED && it > 1 && !mbar_wait(bar(it & 1), ((uint32_t)(it >> 1) & 1u) ^ 1u, 27, abort_flag, p.status)) break;
        tc_fence_after();
        const uint64_t dq_mn = umma_smem_desc(sbase + C::OFF_Q + st * C::TILE_BYTES, 16384, 1024);
        const uint64_t ddo_mn = umma_smem_desc(sbase + C::OFF_DO + st * C::TILE_BYTES, 16384, 1024);
        // dV += P^T dO, dK += dS^T Q : reduction over 16 query rows per step (2048 bytes further in both tiles)
        if (it == 0) {
          umma_bf16(tmem + C::DV_COL, dp_mn, ddo_mn, idesc_t, 0);
          umma_bf16(tmem + C::DK_COL, dds_mn, dq_mn, idesc_t, 0);
        } else {
          umma_bf16_acc(tmem + C::DV_COL, dp_mn, ddo_mn, idesc_t);
          umma_bf16_acc(tmem + C::DK_COL, dds_mn, dq_mn, idesc_t);
        }
#pragma unroll
        for (int t = 1; t < AB_TILE / 16; ++t) {
          umma_bf16_acc(tmem + C::DV_COL, umma_desc_advance(dp_mn, t * 2048), umma_desc_advance(ddo_mn, t * 2048), idesc_t);
          umma_bf16_acc(tmem + C::DK_COL, umma_desc_advance(dds_mn, t * 2048), umma_desc_advance(dq_mn, t * 2048), idesc_t);
        }
        // dQ = dS K : reduction over 16 kv rows per step
        const uint32_t t_dq = tmem + C::DQ_COL + (uint32_t)(it & 1) * C::DQ_BUF_COLS;
        umma_bf16(t_dq, dds_k, dk_mn, idesc_q, 0);
#pragma unroll
        for (int t = 1; t < AB_TILE / 16; ++t)
          umma_bf16_acc(t_dq, umma_desc_advance(dds_k, (t >> 2) * 16384 + (t & 3) * 32),
                        umma_desc_advance(dk_mn, t * 2048), idesc_q);
        umma_commit(bar(8));                        // dQ ready; P / dS and this Q / dO stage are free
        umma_commit(bar(13 + st));
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warpgroups (warps 2..9)
    const int q4 = warp & 3, half = (warp - 2) >> 2;
    const int row = q4 * 32 + lane;
    const uint32_t t_lane = tmem + ((uint32_t)(q4 * 32) << 16);
    constexpr float LOG2E = 1.4426950408889634f;
    bool ok = true;

    // dQ tile of step `it` -> fp32 accumulator in global memory. Each warp turns its [32 rows][HD/2 columns]
    // part into swizzled [32][32 fp32] boxes in shared memory and one lane hands them to the TMA unit as
    // reduce-add tile stores (several KV tiles add into the same query rows), so the SM issues one bulk
    // operation per 4 KB instead of 256 vector atomics.
    uint8_t* stg = sal + C::OFF_DQS + (warp - 2) * 4096;
    const uint32_t stg_s = sbase + C::OFF_DQS + (warp - 2) * 4096;
    auto flush_dq = [&](int it) {
      const int hq = kvh * rep + it / per_head, qi = j + it % per_head;
      const int y0 = qi * AB_TILE + q4 * 32;                 // first of this warp's 32 query rows
#pragma unroll
      for (int c = 0; c < HD / 2; c += 32) {
        uint32_t r[32];
        tmem_ld32(t_lane + C::DQ_COL + (uint32_t)(it & 1) * C::DQ_BUF_COLS + half * (HD / 2) + c, r);
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // staging box free again
        __syncwarp();
        tmem_ld_wait();
        uint8_t* rowp = stg + lane * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
          *reinterpret_cast<uint4*>(rowp + ((ch ^ (lane & 7)) << 4)) = make_uint4(r[4 * ch], r[4 * ch + 1], r[4 * ch + 2], r[4 * ch + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (y0 < p.T && half * (HD / 2) + c < p.hd)
            asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                         ::"l"((uint64_t)&tm_dq), "r"(stg_s), "r"(half * (HD / 2) + c), "r"(y0), "r"(b * p.Hq + hq) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(C::PIPELINED ? bar(it & 1) : bar(9));
    };

    for (int it = 0; it < n_it; ++it) {
      const uint32_t par = (uint32_t)it & 1u;
      const int hq = kvh * rep + it / per_head, qi = j + it % per_head;
      const int t_row = qi * AB_TILE + row;
      const bool row_ok = t_row < p.T;
      const float lse2 = row_ok ? p.lse[((long long)b * p.Hq + hq) * p.T + t_row] * LOG2E : INFINITY;
      const float dlt = row_ok ? p.delta[((long long)b * p.Hq + hq) * p.T + t_row] : 0.f;
      const bool diag = (qi == j);
      if (!mbar_wait(bar(5), par, 28, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
      uint32_t pp[32], dd[32];                      // 64 columns of P and dS, packed bf16 pairs
#pragma unroll
      for (int c = 0; c < 64; c += 32) {
        uint32_t s[32], dp[32];
        tmem_ld32(t_lane + C::S_COL + half * 64 + c, s);
        tmem_ld32(t_lane + C::DP_COL + half * 64 + c, dp);
        tmem_ld_wait();
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(-lse2, -lse2), nd2 = make_float2(-dlt, -dlt);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 x = ffma2(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), sc2, nl2);
          float2 pr = make_float2(ex2_approx(x.x), ex2_approx(x.y));
          if (diag) {
            const int col = half * 64 + c + i;
            if (col > row) pr.x = 0.f;
            if (col + 1 > row) pr.y = 0.f;
          }
          // dS = P (dP - delta); the softmax scale is applied once, when dQ and dK leave their accumulators
          const float2 ds = fmul2(pr, fadd2(make_float2(__uint_as_float(dp[i]), __uint_as_float(dp[i + 1])), nd2));
          pp[(c + i) >> 1] = pack_bf16(pr.x, pr.y);
          dd[(c + i) >> 1] = pack_bf16(ds.x, ds.y);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(6));           // S / dP columns may be overwritten
      if (it > 0) {                                 // MMAs of step it-1 done: P / dS free, dQ(it-1) ready
        if (!mbar_wait(bar(8), par ^ 1u, 29, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
      }
      uint8_t* prow = sal + C::OFF_P + half * 16384 + row * 128;
      uint8_t* drow = sal + C::OFF_DS + half * 16384 + row * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const int sw = (ch ^ (row & 7)) << 4;
        *reinterpret_cast<uint4*>(prow + sw) = make_uint4(pp[4 * ch], pp[4 * ch + 1], pp[4 * ch + 2], pp[4 * ch + 3]);
        *reinterpret_cast<uint4*>(drow + sw) = make_uint4(dd[4 * ch], dd[4 * ch + 1], dd[4 * ch + 2], dd[4 * ch + 3]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(7));
      if (C::PIPELINED) {
        if (it > 0) flush_dq(it - 1);
      } else {
        if (!mbar_wait(bar(8), par, 30, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        flush_dq(it);
      }
    }
    if (ok && n_it > 0) {
      if (C::PIPELINED) {
        if (mbar_wait(bar(8), (uint32_t)(n_it - 1) & 1u, 31, abort_flag, p.status)) { tc_fence_after(); flush_dq(n_it - 1); } else ok = false;
      }
      if (ok) {
        if constexpr (SCATTER) {
          // dV, dK accumulators -> bf16 rows of the packed gradient tensor
          tc_fence_after();
          const int t_row = j * AB_TILE + row;
  #pragma unroll
          for (int which = 0; which < 2; ++which) {
            const int head = which == 0 ? p.Hq + p.Hkv + kvh : p.Hq + kvh;
            const float osc = which == 0 ? 1.f : p.scale;
            const uint32_t col0 = (which == 0 ? C::DV_COL : C::DK_COL) + half * (HD / 2);
            __nv_bfloat16* dst = p.dqkv + (((long long)b * p.T + t_row) * heads_total + head) * p.hd + half * (HD / 2);
            bool dst_ok = true;
            if (p.n_dst > 0) {
              const int owner = t_row / p.dst_rows, tl = t_row - owner * p.dst_rows;
              dst_ok = owner < p.n_dst;
              if (dst_ok)
                dst = p.dst[owner] + (((long long)b * p.dst_rows + tl) * p.dst_heads + (which == 0 ? p.dst_v0 : p.dst_k0) + kvh) * p.hd
                      + half * (HD / 2);
            }
  #pragma unroll
            for (int c = 0; c < HD / 2; c += 32) {
              uint32_t r[32];
              tmem_ld32(t_lane + col0 + c, r);
              tmem_ld_wait();
              // transposed RoPE on dK (fp32): column j pairs with j +- hd / 2. `rot` is warp-uniform (the
              // tensor-memory load of the partner columns must be executed by the whole warp).
              const int colg = half * (HD / 2) + c;                      // first of this thread's 32 columns
              const bool rot = which == 1 && p.cosT != nullptr && colg < p.hd;
              uint32_t q2[32];
              if (rot && p.hd == HD) {                                   // partner columns sit in the other half-row
                tmem_ld32(t_lane + C::DK_COL + (1 - half) * (HD / 2) + c, q2);
                tmem_ld_wait();
              }
              if (rot && t_row < p.T) {
                const float* cr = p.cosT + (long long)t_row * p.hd;
                const float* sr = p.sinT + (long long)t_row * p.hd;
                if (p.hd == HD) {
                  const int pc = (1 - half) * (HD / 2) + c;             // partner's first column
  #pragma unroll
                  for (int i = 0; i < 32; ++i) {
                    const float a = __uint_as_float(r[i]), bb = __uint_as_float(q2[i]);
                    r[i] = __float_as_uint(half == 0 ? a * cr[colg + i] + bb * sr[pc + i] : a * cr[colg + i] - bb * sr[pc + i]);
                  }
                } else {                                                // hd 32 on the 64-wide kernel: both halves are in r
                  float o[32];
  #pragma unroll
                  for (int i = 0; i < 16; ++i) {
                    const float a = __uint_as_float(r[i]), bb = __uint_as_float(r[i + 16]);
                    o[i] = a * cr[i] + bb * sr[i + 16];
                    o[i + 16] = bb * cr[i + 16] - a * sr[i];
                  }
  #pragma unroll
                  for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(o[i]);
                }
              }
              if (t_row < p.T && dst_ok && half * (HD / 2) + c < p.hd) {
  #pragma unroll
                for (int i = 0; i < 32; i += 8) {
                  uint4 v;
                  v.x = pack_bf16(__uint_as_float(r[i]) * osc, __uint_as_float(r[i + 1]) * osc);
                  v.y = pack_bf16(__uint_as_float(r[i + 2]) * osc, __uint_as_float(r[i + 3]) * osc);
                  v.z = pack_bf16(__uint_as_float(r[i + 4]) * osc, __uint_as_float(r[i + 5]) * osc);
                  v.w = pack_bf16(__uint_as_float(r[i + 6]) * osc, __uint_as_float(r[i + 7]) * osc);
                  *reinterpret_cast<uint4*>(dst + c + i) = v;
                }
              }
            }
          }

        } else {
          // dV, dK accumulators -> bf16 rows of the packed gradient tensor
          tc_fence_after();
          const int t_row = j * AB_TILE + row;
  #pragma unroll
          for (int which = 0; which < 2; ++which) {
            const int head = which == 0 ? p.Hq + p.Hkv + kvh : p.Hq + kvh;
            const float osc = which == 0 ? 1.f : p.scale;
            const uint32_t col0 = (which == 0 ? C::DV_COL : C::DK_COL) + half * (HD / 2);
            __nv_bfloat16* dst = p.dqkv + (((long long)b * p.T + t_row) * heads_total + head) * p.hd + half * (HD / 2);
  #pragma unroll
            for (int c = 0; c < HD / 2; c += 32) {
              uint32_t r[32];
              tmem_ld32(t_lane + col0 + c, r);
              tmem_ld_wait();
              if (t_row < p.T && half * (HD / 2) + c < p.hd) {
  #pragma unroll
                for (int i = 0; i < 32; i += 8) {
                  uint4 v;
                  v.x = pack_bf16(__uint_as_float(r[i]) * osc, __uint_as_float(r[i + 1]) * osc);
                  v.y = pack_bf16(__uint_as_float(r[i + 2]) * osc, __uint_as_float(r[i + 3]) * osc);
                  v.z = pack_bf16(__uint_as_float(r[i + 4]) * osc, __uint_as_float(r[i + 5]) * osc);
                  v.w = pack_bf16(__uint_as_float(r[i + 6]) * osc, __uint_as_float(r[i + 7]) * osc);
                  *reinterpret_cast<uint4*>(dst + c + i) = v;
                }
              }
            }
          }

        }
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // dQ reductions have left shared memory and landed
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

template <int HD, bool SCATTER>
static int launch_bwd(const CUtensorMap& mq, const CUtensorMap& mdo, const CUtensorMap& mdq, const AttnBwdParams& p,
                      cudaStream_t st) {
  using C = AttnBwdCfg<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<HD, SCATTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int grid = ((p.T + AB_TILE - 1) / AB_TILE) * p.B * p.Hkv;
  attn_bwd_kernel<HD, SCATTER><<<grid, AB_THREADS, C::TOTAL, st>>>(mq, mdo, mdq, p);
  count_launch();
  return launch_status();
}

}  // namespace tlm

using namespace tlm;

// dq_acc: fp32 scratch [B,Hq,T,hd]; delta: fp32 scratch [B,Hq,T]. Both are owned by the caller.
// cosT / sinT (optional, fp32 [T, hd]): the transposed RoPE is applied to dQ and dK on the way out.
// dst_ptrs (optional, n_dst > 0): head -> sequence return, see AttnBwdParams; dqkv may then be null.
static int attn_bwd_impl(const void* qkv, const void* o, const void* dout, const float* lse, void* dqkv,
                         float* dq_acc, float* delta, int B, int T, int Hq, int Hkv, int hd, float scale,
                         const float* cosT, const float* sinT, void* const* dst_ptrs, int n_dst, int dst_rows,
                         int dst_heads, int dst_q0, int dst_k0, int dst_v0, cudaStream_t st) {
  if (hd != 32 && hd != 64 && hd != 128) return -4;
  if (Hq % Hkv != 0) return -5;
  const long long rows = (long long)B * T * Hq;
  if ((size_t)Hq * (DELTA_T + 1) * 4 > 48 * 1024) return -6;
  attn_delta_kernel<<<B * ((T + DELTA_T - 1) / DELTA_T), DELTA_THREADS, (size_t)Hq * (DELTA_T + 1) * 4, st>>>(
      (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, T, Hq, hd);
  count_launch();
  cudaError_t ce = cudaMemsetAsync(dq_acc, 0, (size_t)rows * hd * 4, st);
  if (ce != cudaSuccess) return (int)ce;
  CUtensorMap mq, mdo;
  int e = make_qkv_map(&mq, qkv, B, T, Hq + 2 * Hkv, hd, AB_TILE);
  if (e) return e;
  e = make_qkv_map(&mdo, dout, B, T, Hq, hd, AB_TILE);
  if (e) return e;
  if ((cosT == nullptr) != (sinT == nullptr)) return -6;
  if (n_dst < 0 || n_dst > AB_MAX_DST || (n_dst > 0 && (dst_ptrs == nullptr || dst_rows <= 0 || (long long)dst_rows * n_dst < T)))
    return -6;
  if (n_dst == 0 && dqkv == nullptr) return -6;
  AttnBwdParams p{};
  p.dqkv = (__nv_bfloat16*)dqkv; p.dq_acc = dq_acc; p.lse = lse; p.delta = delta; p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.status = status_word(); p.hd = hd; p.cosT = cosT; p.sinT = sinT;
  p.n_dst = n_dst; p.dst_rows = dst_rows; p.dst_heads = dst_heads; p.dst_q0 = dst_q0; p.dst_k0 = dst_k0; p.dst_v0 = dst_v0;
  // per (batch, KV head): Q, dO, dQ (fp32 accumulator + bf16 result) of its query heads, K, V, dK, dV; measured at
  // B 8, T 4096, 16 / 8 heads of 64: 1.054 ms with groups of 8 - 16, 1.105 with each head's tiles adjacent, 1.12 with all 64
  p.head_group = attn_head_group("TLM_ATTN_BWD_GROUP", (long long)T * hd * (10LL * (Hq / Hkv) + 8), 112LL << 20, B * Hkv);
  AttnBwdDst dd{};
  dd.n = n_dst; dd.rows = dst_rows; dd.heads = dst_heads;
  for (int i = 0; i < n_dst; ++i) { p.dst[i] = (__nv_bfloat16*)dst_ptrs[i]; dd.p[i] = p.dst[i]; }
  CUtensorMap mdq;                                     // fp32 [B*Hq, T, hd] accumulator, box 32 x 32 x 1
  {
    uint64_t dims[3] = {(uint64_t)hd, (uint64_t)T, (uint64_t)B * Hq};
    uint64_t strides[2] = {(uint64_t)hd * 4, (uint64_t)T * hd * 4};
    uint32_t box[3] = {32, 32, 1};
    e = make_tmap_f32(&mdq, dq_acc, 3, dims, strides, box);
    if (e) return e;
  }
  if (n_dst > 0) e = hd == 128 ? launch_bwd<128, true>(mq, mdo, mdq, p, st) : launch_bwd<64, true>(mq, mdo, mdq, p, st);
  else e = hd == 128 ? launch_bwd<128, false>(mq, mdo, mdq, p, st) : launch_bwd<64, false>(mq, mdo, mdq, p, st);
  if (e) return e;
  // without a return scatter the main kernel has written un-rotated dK into dqkv: this pass rotates it in place
  const int rot_k = (n_dst == 0 && cosT != nullptr) ? Hkv : 0;
  long long items = (long long)B * T * (Hq + rot_k) * (hd / 16);
  int cb = (int)((items + 255) / 256);
  if (cb > num_sms() * 16) cb = num_sms() * 16;
  attn_dq_convert_kernel<<<cb, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dqkv, B, T, Hq, Hq + 2 * Hkv, hd, scale, cosT, sinT, dd, dst_q0,
                                             rot_k);
  count_launch();
  return launch_status();
}

TLM_API int tlm_attn_bwd(const void* qkv, const void* o, const void* dout, const float* lse, void* dqkv,
                         float* dq_acc, float* delta, int B, int T, int Hq, int Hkv, int hd, float scale,
                         const float* cosT, const float* sinT, cudaStream_t st) {
  return attn_bwd_impl(qkv, o, dout, lse, dqkv, dq_acc, delta, B, T, Hq, Hkv, hd, scale, cosT, sinT, nullptr, 0, 0, 0, 0, 0, 0, st);
}

// Attention backward whose gradient rows leave for the sequence owners' packed buffers (see AttnBwdParams):
// dst_ptrs[r]: bf16 [B, dst_rows, dst_heads, hd] on rank r; q slot s -> head dst_q0 + s, k -> dst_k0 + s, v -> dst_v0 + s.
TLM_API int tlm_attn_bwd_scatter(const void* qkv, const void* o, const void* dout, const float* lse, float* dq_acc,
                                 float* delta, int B, int T, int Hq, int Hkv, int hd, float scale, const float* cosT,
                                 const float* sinT, void* const* dst_ptrs, int n_dst, int dst_rows, int dst_heads,
                                 int dst_q0, int dst_k0, int dst_v0, cudaStream_t st) {
  if (n_dst < 1) return -6;
  return attn_bwd_impl(qkv, o, dout, lse, nullptr, dq_acc, delta, B, T, Hq, Hkv, hd, scale, cosT, sinT, dst_ptrs, n_dst,
                       dst_rows, dst_heads, dst_q0, dst_k0, dst_v0, st);
}
