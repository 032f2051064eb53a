// Causal GQA flash attention, forward, on tcgen05 / TMEM.
//
// Input is the packed projection output  qkv[B, T, Hq + 2*Hkv, hd]  (bf16):
// heads [0,Hq) are queries, [Hq,Hq+Hkv) keys, [Hq+Hkv,Hq+2Hkv) values; query
// head h reads KV head h / (Hq/Hkv) in place, nothing is expanded or transposed.
// Output o[B, T, Hq, hd] (bf16) and lse[B, Hq, T] (fp32, natural log).
//
// One CTA owns 128 query rows of one (batch, head) and walks over 128-row KV
// tiles up to the diagonal:
//   warp 0     TMA: Q once, then K / V tiles into a 2-deep ring (128B swizzle)
//   warp 1     one lane issues  S = Q K^T  (M128 N128) into TMEM, and after the
//              softmax warps have published P:  O_j = P V  (M128 N=hd; V is
//              consumed as an MN-major operand straight from its row-major tile)
//   warps 2-5  one thread per query row: tcgen05.ld S, running max / sum with
//              exp2, P written back to tensor memory as packed bf16 pairs (the A
//              operand of the P V MMA). O accumulates in TMEM across KV tiles; it is only
//              rescaled (ld / multiply / st) when the row maximum grew by more
//              than 2^8, and S of tile j+1 is issued while tile j's softmax runs
// Shared memory is 80 KB and tensor memory 256 columns (hd 64), so two CTAs share an
// SM and one CTA's softmax overlaps the other's MMAs. All waits are bounded.
#include "common.cuh"

namespace tlm {

constexpr int AT_BQ = 128, AT_BKV = 128, AT_THREADS = 192, AT_KV_STAGES = 2;

constexpr int AT_MAX_DST = 8;

struct AttnFwdParams {
  __nv_bfloat16* o;
  float* lse;
  int B, T, Hq, Hkv;
  float scale_log2;        // softmax scale * log2(e)
  float scale;             // softmax scale
  unsigned int* status;
  // Optional second copy of the output for sequence parallelism (head -> sequence exchange done by
  // this kernel's epilogue): row t of head h also goes to
  //   o_dst[t / dst_rows][b, t % dst_rows, dst_head0 + h, :]   (bf16 [B, dst_rows, dst_heads, hd] per rank;
  // peer-mapped addresses, plain 16-byte stores). n_dst == 0 disables it.
  __nv_bfloat16* o_dst[AT_MAX_DST];
  int n_dst, dst_rows, dst_heads, dst_head0;
  // Head dim of the tensors in memory. It equals the kernel's HD except for hd = 32, which runs on the
  // HD = 64 kernel: the TMA boxes stay 64 wide and the 32 columns past the end of a head are
  // out-of-bounds zero fill, so Q K^T is unchanged and the upper half of O is never stored.
  int hd;
  int head_group;          // heads per group of the heavy-first block order (see heavy_first_decode)
};

template <int HD>
struct AttnFwdSmem {
  static constexpr int KB = HD / 64;                   // 64-wide blocks along hd
  static constexpr int Q_BYTES = AT_BQ * HD * 2;
  static constexpr int KV_BYTES = AT_BKV * HD * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + AT_KV_STAGES * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + AT_KV_STAGES * KV_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256;          // + barriers; 2 CTAs (hd 64) must fit in 228 KB
};

// Thread `row` owns one query row: running reference max `m_ref`, running sum `l_run`.
// The exponent reference is only moved (and O rescaled in TMEM) when the tile
// maximum exceeds it by more than RESCALE_LOG2 in the log2 domain, so most tiles
// do no rescaling; the result is exact either way because the same reference
// is used for P and for the final normalisation.
constexpr float RESCALE_LOG2 = 8.0f;

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, HD == 64 ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, const AttnFwdParams p) {
  using L = AttnFwdSmem<HD>;
  constexpr int KB = L::KB;
  // tensor-memory columns: S (128 fp32), O (HD fp32) and the probabilities as packed bf16 pairs (64 columns),
  // which the P V MMA reads as its A operand straight from tensor memory (P never touches shared memory)
  constexpr uint32_t S_COL = 0, O_COL = 128, P_COL = 128 + HD;
  constexpr uint32_t TMEM_COLS = HD == 128 ? 512 : 256;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t sbase = smem_u32(smem_raw);
  uint8_t* sal = smem_raw;
  if (sbase & 1023u) {                                // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) report_status(p.status, (10u << 8) | 2u);
    return;
  }
  const uint32_t bar0 = sbase + L::OFF_BAR;
  // barriers: 0 q_full, 1..2 k_full, 3..4 v_full, 5..6 v_empty, 7 s_full, 8 p_full, 9 o_done, 10 s_consumed,
  //           11..12 k_empty. A K stage is free as soon as its S = Q K^T has run, long before the stage's V is
  //           consumed, so K tiles are loaded one step ahead of V tiles and their latency stays hidden.
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sal + L::OFF_BAR + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_q_tiles = (p.T + AT_BQ - 1) / AT_BQ;
  int tile_rank, bh;
  heavy_first_decode((int)blockIdx.x, n_q_tiles, p.B * p.Hq, p.head_group, tile_rank, bh);
  const int qt = n_q_tiles - 1 - tile_rank;           // heavy (late) tiles first
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  const int q0 = qt * AT_BQ;
  const int n_kv = qt + 1;                            // causal: KV tiles 0..qt

  if (threadIdx.x == 0) {
    for (int i = 0; i < 13; ++i) mbar_init(bar(i), (i == 8 || i == 10) ? 4 : 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_qkv);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(0), L::Q_BYTES);
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) tma_load_4d(sbase + L::OFF_Q + kb * 16384, &tm_qkv, bar(0), kb * 64, h, q0, b);
      auto load_k = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(bar(11 + st), ((uint32_t)(j >> 1) & 1u) ^ 1u, 11, abort_flag, p.status)) return false;
        mbar_expect_tx(bar(1 + st), L::KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_4d(sbase + L::OFF_K + st * L::KV_BYTES + kb * 16384, &tm_qkv, bar(1 + st), kb * 64, p.Hq + kvh, j * AT_BKV, b);
        return true;
      };
      bool ok = load_k(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < n_kv && !load_k(j + 1)) break;
        if (!mbar_wait(bar(5 + st), ((uint32_t)(j >> 1) & 1u) ^ 1u, 20, abort_flag, p.status)) break;
        mbar_expect_tx(bar(3 + st), L::KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_4d(sbase + L::OFF_V + st * L::KV_BYTES + kb * 16384, &tm_qkv, bar(3 + st), kb * 64, p.Hq + p.Hkv + kvh, j * AT_BKV, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(AT_BQ, AT_BKV, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(AT_BQ, HD, 0, 1);
      // descriptors are built once per tile and advanced with one add per MMA: this thread's instruction
      // stream is what feeds the tensor pipe
      const uint64_t dq = umma_smem_desc(sbase + L::OFF_Q, 16, 1024);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(bar(1 + st), (uint32_t)(j >> 1) & 1u, 13, abort_flag, p.status)) return false;
        tc_fence_after();
        const uint64_t dk = umma_smem_desc(sbase + L::OFF_K + st * L::KV_BYTES, 16, 1024);
        umma_bf16(tmem + S_COL, dq, dk, idesc_s, 0);
#pragma unroll
        for (int t = 1; t < HD / 16; ++t) {
          const uint32_t off = (t >> 2) * 16384 + (t & 3) * 32;
          umma_bf16_acc(tmem + S_COL, umma_desc_advance(dq, off), umma_desc_advance(dk, off), idesc_s);
        }
        umma_commit(bar(7));
        umma_commit(bar(11 + st));                              // K stage free
        return true;
      };
      bool ok = mbar_wait(bar(0), 0, 12, abort_flag, p.status);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t par = (uint32_t)j & 1u;
        if (j + 1 < n_kv) {                                     // S of the next tile overlaps this tile's softmax
          if (!mbar_wait(bar(10), par, 18, abort_flag, p.status)) break;
          if (!issue_s(j + 1)) break;
        }
        if (!mbar_wait(bar(8), par, 14, abort_flag, p.status)) break;                        // P written
        if (!mbar_wait(bar(3 + st), (uint32_t)(j >> 1) & 1u, 15, abort_flag, p.status)) break;   // V landed
        tc_fence_after();
        const uint64_t dv = umma_smem_desc(sbase + L::OFF_V + st * L::KV_BYTES, 16384, 1024);   // MN-major: 16 kv rows per step
#pragma unroll
        for (int t = 0; t < AT_BKV / 16; ++t)                   // 16 kv = 8 columns of packed pairs per step
          umma_bf16_ts(tmem + O_COL, tmem + P_COL + t * 8, umma_desc_advance(dv, t * 2048), idesc_o, (j > 0) | (t > 0));
        umma_commit(bar(9));                                    // O updated, P free
        umma_commit(bar(5 + st));                               // V stage free
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;                              // row inside the tile == TMEM lane
    const uint32_t t_lane = tmem + ((uint32_t)(q * 32) << 16);
    const float tau = RESCALE_LOG2 / p.scale_log2;              // threshold in raw-score units
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const uint32_t par = (uint32_t)j & 1u;
      if (!mbar_wait(bar(7), par, 16, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
      const bool diag = (j == qt);
      // ---- the whole S row (128 fp32) moves to registers in one go; S may then be overwritten by the next
      // tile's Q K^T, which therefore overlaps all of this tile's softmax
      uint32_t sr[AT_BKV];
#pragma unroll
      for (int c = 0; c < AT_BKV; c += 32) tmem_ld32(t_lane + S_COL + c, sr + c);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(10));
      // ---- row maximum
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      if (!diag) {
#pragma unroll
        for (int i = 0; i < AT_BKV; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(sr[i]));     mx1 = fmaxf(mx1, __uint_as_float(sr[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(sr[i + 2])); mx3 = fmaxf(mx3, __uint_as_float(sr[i + 3]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < AT_BKV; ++i) if (i <= row) mx0 = fmaxf(mx0, __uint_as_float(sr[i]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      // ---- the reference only moves when the maximum grew a lot (O is then rescaled below)
      const bool grow = j > 0 && mx > m_ref + tau;
      float alpha = 1.f;
      if (j == 0) m_ref = mx;
      else if (grow) { alpha = ex2_approx((m_ref - mx) * p.scale_log2); m_ref = mx; }
      const float neg_m = -m_ref * p.scale_log2;
      // ---- probabilities as packed bf16 pairs, still in registers (they take the place of the S row)
      float2 l2 = make_float2(0.f, 0.f);
      const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(neg_m, neg_m);
      uint32_t pk[AT_BKV / 2];
#pragma unroll
      for (int i = 0; i < AT_BKV; i += 2) {
        const float2 x = ffma2(make_float2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), sc2, nm2);
        float2 pp = make_float2(ex2_approx(x.x), ex2_approx(x.y));
        if (diag) { if (i > row) pp.x = 0.f; if (i + 1 > row) pp.y = 0.f; }
        l2 = fadd2(l2, pp);
        pk[i >> 1] = pack_bf16(pp.x, pp.y);
      }
      // ---- only now is the previous tile's P V needed to be complete (P is overwritten, O may be rescaled):
      // by this time it is, so the wait costs nothing
      if (j > 0) {
        if (!mbar_wait(bar(9), par ^ 1u, 17, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
          for (int c = 0; c < HD; c += 8) {                    // rare path; narrow chunks keep registers free
            uint32_t r[8];
            tmem_ld8(t_lane + O_COL + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st8(t_lane + O_COL + c, r);
          }
        }
      }
      l_run = fmaf(l_run, alpha, l2.x + l2.y);
#pragma unroll
      for (int c = 0; c < AT_BKV; c += 32)
        tmem_st16(t_lane + P_COL + (c >> 1), pk + (c >> 1));    // word i of the row = probabilities 2i, 2i+1
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(8));
    }
    if (ok) ok = mbar_wait(bar(9), (uint32_t)(n_kv - 1) & 1u, 19, abort_flag, p.status);
    const int t_row = q0 + row;
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l_run;
      __nv_bfloat16* out = p.o + (((long long)b * p.T + t_row) * p.Hq + h) * p.hd;
      __nv_bfloat16* out2 = nullptr;
      if (p.n_dst > 0 && t_row < p.T) {
        const int dest = t_row / p.dst_rows, tl = t_row - dest * p.dst_rows;
        if (dest < p.n_dst) out2 = p.o_dst[dest] + (((long long)b * p.dst_rows + tl) * p.dst_heads + p.dst_head0 + h) * p.hd;
      }
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t r[32];
        tmem_ld32(t_lane + O_COL + c, r);
        tmem_ld_wait();
        if (t_row < p.T && c < p.hd) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
            *reinterpret_cast<uint4*>(out + c + i) = v;
            if (out2 != nullptr) *reinterpret_cast<uint4*>(out2 + c + i) = v;
          }
        }
      }
      if (t_row < p.T) p.lse[((long long)b * p.Hq + h) * p.T + t_row] = m_ref * p.scale + __logf(l_run);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// 4-D map over the packed tensor: dims (hd, heads, T, B); box (64, 1, rows, 1). For hd = 32 the box is wider
// than the tensor's inner extent; the excess columns are zero fill.
int make_qkv_map(CUtensorMap* map, const void* base, int B, int T, int heads, int hd, int box_rows) {
  uint64_t dims[4] = {(uint64_t)hd, (uint64_t)heads, (uint64_t)T, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)hd * 2, (uint64_t)heads * hd * 2, (uint64_t)T * heads * hd * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_tmap_bf16(map, base, 4, dims, strides, box);
}

template <int HD>
static int launch_fwd(const CUtensorMap& map, const AttnFwdParams& p, cudaStream_t st) {
  using L = AttnFwdSmem<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int grid = ((p.T + AT_BQ - 1) / AT_BQ) * p.B * p.Hq;
  attn_fwd_kernel<HD><<<grid, AT_THREADS, L::TOTAL, st>>>(map, p);
  count_launch();
  return launch_status();
}

}  // namespace tlm

using namespace tlm;

static int attn_fwd_impl(const void* qkv, void* o, float* lse, int B, int T, int Hq, int Hkv, int hd, float scale,
                         void* const* o_dst, int n_dst, int dst_rows, int dst_heads, int dst_head0, cudaStream_t st) {
  if (hd != 32 && hd != 64 && hd != 128) return -4;
  if (Hq % Hkv != 0) return -5;
  if (n_dst < 0 || n_dst > AT_MAX_DST || (n_dst > 0 && (dst_rows <= 0 || (long long)dst_rows * n_dst < T))) return -6;
  CUtensorMap map;
  int e = make_qkv_map(&map, qkv, B, T, Hq + 2 * Hkv, hd, AT_BQ);
  if (e) return e;
  AttnFwdParams p{};
  p.o = (__nv_bfloat16*)o; p.lse = lse; p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.scale_log2 = scale * 1.4426950408889634f; p.scale = scale; p.status = status_word();
  p.n_dst = n_dst; p.dst_rows = dst_rows; p.dst_heads = dst_heads; p.dst_head0 = dst_head0; p.hd = hd;
  for (int i = 0; i < n_dst; ++i) p.o_dst[i] = (__nv_bfloat16*)o_dst[i];
  // a head's Q, K, V and O rows; in-step timing at B 8, T 4096, 16 heads of 64: groups of 16 - 32 heads are best
  // (0.45 ms against 0.49 ms with each head's tiles adjacent), all 128 heads at once lose that again to L2 misses
  p.head_group = attn_head_group("TLM_ATTN_FWD_GROUP", 8LL * T * hd, 48LL << 20, B * Hq);
  return hd == 128 ? launch_fwd<128>(map, p, st) : launch_fwd<64>(map, p, st);
}

TLM_API int tlm_attn_fwd(const void* qkv, void* o, float* lse, int B, int T, int Hq, int Hkv, int hd, float scale,
                         cudaStream_t st) {
  return attn_fwd_impl(qkv, o, lse, B, T, Hq, Hkv, hd, scale, nullptr, 0, 0, 0, 0, st);
}

// Same, and the epilogue also stores every output row into the memory of the rank that owns the
// row's sequence chunk (see AttnFwdParams): the head -> sequence exchange of Ulysses sequence parallelism.
TLM_API int tlm_attn_fwd_scatter(const void* qkv, void* o, float* lse, int B, int T, int Hq, int Hkv, int hd,
                                 float scale, void* const* o_dst, int n_dst, int dst_rows, int dst_heads,
                                 int dst_head0, cudaStream_t st) {
  return attn_fwd_impl(qkv, o, lse, B, T, Hq, Hkv, hd, scale, o_dst, n_dst, dst_rows, dst_heads, dst_head0, st);
}
