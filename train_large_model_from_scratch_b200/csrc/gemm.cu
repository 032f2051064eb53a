// Persistent, warp-specialised bf16 GEMM on the 5th-generation tensor cores.
//
//   C[M,N] (=|+=) A[M,K] * B[N,K]^T      fp32 accumulation in tensor memory
//
// One CTA per SM walks over 128x256 output tiles. Roles inside the CTA:
//   warp 0      : TMA producer - fills a 4-deep ring of (A 128x64, B 256x64) bf16
//                 stages in 128B-swizzled shared memory
//   warp 1      : allocates 512 TMEM columns (two 128x256 fp32 accumulators) and,
//                 through one elected lane, issues tcgen05.mma (M128 N256 K16)
//   warps 2..5  : epilogue - tcgen05.ld the finished accumulator (each warp owns
//                 the 32 TMEM lanes its rank allows), convert, store to global
// The two accumulators let the MMA warp start tile i+1 while the epilogue
// drains tile i.
//
// Either operand may be "K-major" (reduction index contiguous in memory:
// A stored [M,K], B stored [N,K]) or "MN-major" (output index contiguous:
// A stored [K,M], B stored [K,N]). The major-ness only changes the TMA boxes
// and two descriptor fields, so forward (x W^T), dgrad (dy W) and wgrad
// (dy^T x, accumulated into the fp32 gradient buffer) all run on this kernel
// without transposed copies.
//
// Every mbarrier wait is bounded; on a timeout the CTA records a status code,
// every role leaves its loop, and the CTA still frees its tensor memory.
#include "common.cuh"
#include <cuda_fp16.h>

namespace tlm {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;                 // 16 KB
constexpr int B_BYTES = BN * BK * 2;                 // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int BOX_MN_BYTES = 64 * BK * 2;            // one 64(mn) x 64(k) MN-major box = 8 KB
constexpr int TMEM_COLS = 512;
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_THREADS_WIDE = 320;               // 8 epilogue warps (two per TMEM lane quarter) for the heavy epilogue
constexpr int EPI_BUF_BYTES = 32 * 128;              // one warp's 32 rows x 64 bf16 staging tile
constexpr int EPI_BYTES = 4 * 2 * EPI_BUF_BYTES;     // 4 epilogue warps x 2 buffers = 32 KB
constexpr int GEMM_SMEM = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
// CTA pairs (see gemm_body, PAIR): each CTA stages its own 128 rows of A and HALF of the tile's B rows, so a stage is
// 32 KB per CTA and the ring is six stages deep.
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_STAGE_BYTES = A_BYTES + B_BYTES / 2;
constexpr int GEMM_SMEM_PAIR = PAIR_STAGES * PAIR_STAGE_BYTES + EPI_BYTES + 1024 + 256;

enum Epilogue { EPI_BF16 = 0, EPI_F32_ACC = 1, EPI_F32 = 2, EPI_HEADS = 3, EPI_SWIGLU = 4, EPI_SWIGLU_BWD = 5, EPI_LSE = 6,
                EPI_ROWS = 7 /* bf16 rows stored at looked-up (buffer, row): the expert-parallel combine */ };

// Destinations of the head-scatter epilogue: one 4-D map (hd, heads, T, B; box 64 x 1 x 32 x 1)
// per rank of the sequence-parallel group; entry 0 alone when the output stays local.
constexpr int MAX_HEAD_DST = 8;
struct HeadDstMaps { CUtensorMap m[MAX_HEAD_DST]; };

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;            // elements
  unsigned int* status;
  // grouped mode (MoE): problem g covers rows [row_start[g], row_start[g+1]) of a
  // row-grouped operand; see grouped launchers. groups == 0 -> plain GEMM.
  int groups;
  const int* row_start;     // device, groups + 1 entries
  int group_mode;           // 1: rows of A/C grouped, B per group (3-D map); 2: K grouped (wgrad), C per group
  long long c_group_stride; // elements between per-group C matrices (mode 2)
  int max_tiles_m;          // upper bound of m-tiles per group (mode 1)
  int split_k;              // plain GEMM with fp32 accumulate: reduction split into this many tiles (>= 1);
                            // with split_k > 1 the epilogue adds with red.global (order not deterministic)
  int k_chunk;              // reduction length per split (multiple of BK)
  int tma_store;            // bf16 epilogue through shared memory + TMA store (plain GEMM only)
  // EPI_HEADS: the N axis is a run of heads of `hd` columns (q heads, then k, then v) and the M axis is
  // [batch][rows_per_batch]. Head h of row (b, t) is rotated (RoPE, heads < n_rot) and stored as bf16 into
  //   dst[owner(h)][b, row_off + t, slot(h), :]
  // where owner / slot follow the Ulysses head plan: q head h -> (h / q_l, h % q_l), k head j ->
  // (j / kv_l, q_l + j % kv_l), v head j -> (j / kv_l, q_l + kv_l + j % kv_l). With one destination and
  // q_l = Hq, kv_l = Hkv this is the identity layout [B, T, Hq + 2 Hkv, hd].
  // kv_rep > 1 (fewer KV heads than destinations): k / v head j is needed by the kv_rep ranks that own its query
  // heads, so its tile is stored kv_rep times: dst[j * kv_rep + c], slots q_l (k) and q_l + 1 (v), c < kv_rep.
  int hd, rows_per_batch, row_off, Hq, Hkv, q_l, kv_l, n_rot, kv_rep;
  const __half2* cs;        // [rows_per_batch, hd] (cos, sin) pairs in fp16: |error| < 2^-11, below the bf16 rounding of
                            // the rotated outputs, and half the table bytes of two fp32 tables
  // EPI_SWIGLU (MLP forward): B is the fused [2 I, K] weight (gate rows, then up rows), N = I. A tile holds the
  //   SAME 128 columns of gate and of up (two 128-row B boxes), and the epilogue writes three bf16 tiles:
  //   gate and up into C = gate_up [M, 2 I] (kept for backward) and silu(gate) * up into act [M, I].
  // EPI_SWIGLU_BWD (MLP backward): C' = dy W_down is d(act); the epilogue reads gate / up of the same rows and
  //   columns from `aux` ([M, 2 I], row pitch 2 N) and writes d(gate), d(up) into C = d(gate_up) [M, 2 I].
  // Both round their GEMM result to bf16 first, so the numbers equal the separate GEMM + SwiGLU kernels'.
  const __nv_bfloat16* aux;
  // Grouped SwiGLU (MoE experts): rows grouped like group_mode 1, B holds 2 * groups matrices (gate of group g at g,
  // up at groups + g). A tile's rows past its group's end belong to the next group, so warps whose 32 rows cross
  // that end store row by row with a mask instead of with TMA tile stores; `act` / `ld_act` locate the act tensor
  // for those stores.
  __nv_bfloat16* act;
  long long ld_act;
  // EPI_LSE (LM head without logits): nothing of C is stored. Each output row keeps, per 256-column tile, the
  // maximum and the sum of exp(x - max) of its (bf16-rounded) logits in lse_part[row * lse_tiles + tile] and, in the
  // tile that holds the row's target column, the target logit in tgt_logit[row]; a small second kernel folds the
  // tiles into log-sum-exp and loss. The [M, V] logits never exist in memory.
  float2* lse_part;
  int lse_tiles;
  const long long* targets;
  float* tgt_logit;
  // bf16 store with the cross-entropy gradient applied on the way out (dl_lse != nullptr): the tile holds logits x and
  // what is stored is  *dl_scale * (exp(x - dl_lse[row]) - [col == targets[row]])  (0 for rows whose target is
  // dl_ignore). Second pass of the LM head without logits: the gradient tile goes straight to the dgrad / wgrad GEMMs.
  const float* dl_lse;
  const float* dl_scale;
  long long dl_ignore;
  // Paired groups (grouped rows, MoE gate|up): the B map has 2 * groups matrices, gate of group g at g and up at
  // groups + g. pair_n > 0: output columns >= pair_n come from the second matrix (forward: one GEMM writes
  // gate|up [R, 2 I]). pair_k > 0: reduction indices >= pair_k come from the second matrix (dgrad of both
  // projections in one GEMM with K = 2 I, so their sum needs no extra pass).
  int pair_n, pair_k;
  // Row-scatter epilogue (bf16 store, grouped rows): output row r is not written to C but to
  //   rs_dst[rs_rank[r]] + rs_row[r] * ldc   (rows with rs_rank[r] < 0 are dropped).
  // This is the expert-parallel combine: the down-projection's accumulator goes straight to the
  // token owner's buffer (peer-mapped addresses, plain 16-byte stores). rs_rank == nullptr: off.
  const int* rs_rank;
  const long long* rs_row;
  void* rs_dst[MAX_HEAD_DST];
  long long rs_rows;        // rows of a destination buffer (stores outside are refused)
  // "Parameters ready" gate (sharded optimizer, several ranks): before its first TMA load the producer warp waits
  // until every rank's update of the listed buckets has arrived in this rank's parameter replica (flag words in
  // symmetric memory, see READY_* in common.cuh). This is where the parameter all-gather of the previous
  // optimizer step is consumed: the first GEMM that reads a bucket's weights waits for them itself, so no barrier
  // stands between the optimizer step and the next forward pass. wait_flags[i] == nullptr: no gate.
  const int* wait_flags[2];
  int wait_bucket[2], wait_n[2];
};

// Gates armed by tlm_gemm_arm_param_wait; the next GEMM launch of this library takes them all.
static struct { const int* flags; int bucket, n; } g_pending_wait[2];
static int g_n_pending_wait = 0;

static void take_pending_waits(GemmParams& p) {
  for (int i = 0; i < 2; ++i) {
    p.wait_flags[i] = i < g_n_pending_wait ? g_pending_wait[i].flags : nullptr;
    p.wait_bucket[i] = i < g_n_pending_wait ? g_pending_wait[i].bucket : 0;
    p.wait_n[i] = i < g_n_pending_wait ? g_pending_wait[i].n : 0;
  }
  g_n_pending_wait = 0;
}

struct TileCoord {
  int m0, n0;       // output tile origin (row within C / column)
  int a_row0;       // row coordinate for the A operand
  int b_grp;        // third coordinate of the B map (grouped) or 0
  int b_n0;         // row (K-major) / column (MN-major) coordinate of the tile in the B matrix; n0 unless pair_n
  int k_lo, k_hi;   // reduction range
  int m_end;        // exclusive row bound for stores
  long long c_off;  // element offset added to C
  bool valid;
};

__device__ __forceinline__ TileCoord plain_tile(const GemmParams& p, int tile_in, int tiles_m, int tiles_n, int tile_n,
                                                int tile_m = BM, int m_shift = 0) {
  // split-major order: CTAs that run together work on different output tiles, so the red.global passes of
  // the k-splits of one tile do not collide in time
  const int n_out = tiles_m * tiles_n;
  const int ks = tile_in / n_out, tile = tile_in - ks * n_out;
  // bands of 16 row-tiles, column-tiles fastest inside a band -> the CTAs that
  // run together share a handful of A and B tiles in L2
  const int GROUP_M = tile_m == BM ? 16 : 8;        // 2048 rows per band either way
  int band = tile / (GROUP_M * tiles_n);
  int first_m = band * GROUP_M;
  int gm = min(GROUP_M, tiles_m - first_m);
  int r = tile - band * GROUP_M * tiles_n;
  int tm = first_m + r % gm, tn = r / gm;
  TileCoord t;
  t.m0 = tm * tile_m + m_shift; t.n0 = tn * tile_n; t.a_row0 = t.m0; t.b_grp = 0; t.b_n0 = t.n0;
  t.k_lo = ks * p.k_chunk; t.k_hi = min(p.K, t.k_lo + p.k_chunk); t.m_end = p.M; t.c_off = 0; t.valid = t.k_hi > t.k_lo;
  return t;
}

// GATED: the producer warp first waits for the "parameters ready" words listed in p.wait_*. Only the kernels that can
// be the first reader of a bucket's weights (the QKV projection: head-scatter GEMM, plain x W^T) have a gated
// instantiation; every other kernel is compiled without the gate, whose mere presence in the producer warp's
// preamble measurably slows the main loop (3 - 7 % on the weight-gradient shapes).
//
// PAIR: the kernel runs as clusters of two CTAs on one 256 x 256 tile (plain GEMMs only). Rank r of the pair owns
// output rows [128 r, 128 r + 128) of the tile: it loads those rows of A and rows [128 r, +128) of the tile's B
// operand (for the SwiGLU forward: rank 0 the gate rows, rank 1 the up rows) with its own TMA producer, and reads its
// accumulator half from its own tensor memory with its own epilogue warps. Rank 0's MMA lane issues M = 256
// cta_group::2 MMAs that read both CTAs' shared memory, so every CTA pulls 32 KB per k-block out of L2 instead of
// 48 KB. Barriers: `full` lives in rank 0 (both producers' loads complete on it), `empty` and `accumulator full` are
// signalled in both CTAs by the leader's commits, `accumulator empty` lives in rank 0 and collects both CTAs'
// epilogue warps.
template <bool A_MN, bool B_MN, int EPI, bool GATED = false, bool PAIR = false>
__device__ __forceinline__ void gemm_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                                          const GemmParams& p, const CUtensorMap* dst_maps) {
  static_assert(!(PAIR && GATED), "the gated instantiations run as single CTAs");
  constexpr int STAGES = PAIR ? PAIR_STAGES : tlm::STAGES;
  constexpr int B_TILE_BYTES = PAIR ? B_BYTES / 2 : B_BYTES;
  constexpr int STAGE_BYTES = A_BYTES + B_TILE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + STAGES * STAGE_BYTES + EPI_BYTES);
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;        // tile walker id and count
  const int n_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  // barrier slots: full[0..S), empty[S..2S), acc_full[2S..2S+2), acc_empty[2S+2..2S+4)
  const uint32_t bar0 = smem_base + STAGES * STAGE_BYTES + EPI_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto accf_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto acce_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The SwiGLU-backward epilogue reads gate / up from global memory and is as long as the main loop of its
  // K = hidden-size tiles, so it runs on 8 warps: warps 2-5 take the left 128 columns, warps 6-9 the right.
  constexpr int EPI_WARPS = EPI == EPI_SWIGLU_BWD ? 8 : 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(accf_bar(a), 1); mbar_init(acce_bar(a), EPI_WARPS * (PAIR ? 2 : 1)); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish_pair(); }
    else { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all();          // the peer's barriers are initialised before anything signals them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  constexpr int TILE_N = EPI == EPI_SWIGLU ? 128 : BN;      // output columns per tile (SwiGLU: 128 gate + 128 up)
  constexpr int TILE_M = PAIR ? 2 * BM : BM;                // rows per tile walker
  const int tiles_n = (p.N + TILE_N - 1) / TILE_N;
  int tiles_m, total_tiles;
  if (p.groups == 0) { tiles_m = (p.M + TILE_M - 1) / TILE_M; total_tiles = tiles_m * tiles_n * p.split_k; }
  else if (p.group_mode == 1) { tiles_m = p.max_tiles_m; total_tiles = p.groups * tiles_m * tiles_n; }
  else { tiles_m = (p.M + BM - 1) / BM; total_tiles = p.groups * tiles_m * tiles_n; }

  auto get_tile = [&](int tile) -> TileCoord {
    if (p.groups == 0) return plain_tile(p, tile, tiles_m, tiles_n, TILE_N, TILE_M, (int)cta_rank * BM);
    TileCoord t;
    int per = tiles_m * tiles_n;
    int g = tile / per, r = tile - g * per;
    int tm = r % tiles_m, tn = r / tiles_m;
    int lo = p.row_start[g], hi = p.row_start[g + 1];
    if (p.group_mode == 1) {            // rows grouped: A rows [lo,hi), B = weight[g]
      // PAIR: both CTAs of a pair must agree on whether the tile exists, so that is decided on the pair's first row;
      // a second half that starts past the group's end runs with every row masked
      const int m_first = lo + tm * TILE_M;
      t.m0 = m_first + (int)cta_rank * BM; t.a_row0 = t.m0; t.n0 = tn * TILE_N; t.b_grp = g; t.b_n0 = t.n0;
      if (p.pair_n > 0 && t.n0 >= p.pair_n) { t.b_grp = g + p.groups; t.b_n0 = t.n0 - p.pair_n; }
      t.k_lo = 0; t.k_hi = p.K; t.m_end = hi; t.c_off = 0; t.valid = m_first < hi;
    } else {                            // reduction grouped: K range [lo,hi), C = C_base + g * stride
      t.m0 = tm * BM; t.a_row0 = t.m0; t.n0 = tn * BN; t.b_grp = 0; t.b_n0 = t.n0;
      t.k_lo = lo; t.k_hi = hi; t.m_end = p.M; t.c_off = (long long)g * p.c_group_stride; t.valid = hi > lo;
    }
    return t;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    bool gate_ok = true;
    if (GATED) {
      // weights of this GEMM may still be on their way from the ranks that own their optimizer shards
#pragma unroll
      for (int w = 0; w < 2; ++w)
        if (p.wait_flags[w] != nullptr) gate_ok &= wait_params_ready(p.wait_flags[w], p.wait_bucket[w], p.wait_n[w], lane, p.status, 45);
      gate_ok = __all_sync(0xffffffffu, gate_ok);
      if (!gate_ok) *abort_flag = 1;
      asm volatile("fence.proxy.async;" ::: "memory");      // the peers' (generic-proxy) stores before this warp's TMA reads
    }
    if (lane == 0 && (!GATED || gate_ok)) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = worker; tile < total_tiles && ok; tile += n_workers) {
        TileCoord t = get_tile(tile);
        if (!t.valid) continue;
        for (int k0 = t.k_lo; k0 < t.k_hi; k0 += BK) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, 1, abort_flag, p.status)) { ok = false; break; }
          const uint32_t sa = smem_base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          if (PAIR) {
            // both CTAs' loads of this stage complete on the leader's barrier
            const uint32_t fb = mapa_shared(full_bar(stage), 0);
            if (leader) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * BOX_MN_BYTES, &tmA, fb, t.a_row0 + 64 * j, k0);
            } else {
              tma_load_2d_pair(sa, &tmA, fb, k0, t.a_row0);
            }
            const int half_n0 = (int)cta_rank * (BN / 2);       // this CTA's half of the tile's B rows
            int pbk = k0, pbg = t.b_grp;
            if (p.pair_k > 0 && k0 >= p.pair_k) { pbk = k0 - p.pair_k; pbg += p.groups; }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j) tma_load_3d_pair(sb + j * BOX_MN_BYTES, &tmB, fb, t.b_n0 + half_n0 + 64 * j, pbk, pbg);
            } else if (EPI == EPI_SWIGLU) {                     // rank 0: 128 gate rows, rank 1: the matching up rows
              if (p.groups > 0) tma_load_3d_pair(sb, &tmB, fb, k0, t.n0, t.b_grp + (leader ? 0 : p.groups));
              else tma_load_3d_pair(sb, &tmB, fb, k0, (leader ? 0 : p.N) + t.n0, 0);
            } else {
              tma_load_3d_pair(sb, &tmB, fb, pbk, t.b_n0 + half_n0, pbg);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * BOX_MN_BYTES, &tmA, full_bar(stage), t.a_row0 + 64 * j, k0);
          } else {
            tma_load_2d(sa, &tmA, full_bar(stage), k0, t.a_row0);
          }
          int bk = k0, bg = t.b_grp;
          if (p.pair_k > 0 && k0 >= p.pair_k) { bk = k0 - p.pair_k; bg += p.groups; }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(sb + j * BOX_MN_BYTES, &tmB, full_bar(stage), t.b_n0 + 64 * j, bk, bg);
          } else if (EPI == EPI_SWIGLU) {       // 128 gate rows, then the matching 128 up rows
            if (p.groups > 0) {                 // experts: gate matrix of the group, then its up matrix
              tma_load_3d(sb, &tmB, full_bar(stage), k0, t.n0, t.b_grp);
              tma_load_3d(sb + B_BYTES / 2, &tmB, full_bar(stage), k0, t.n0, t.b_grp + p.groups);
            } else {
              tma_load_3d(sb, &tmB, full_bar(stage), k0, t.n0, 0);
              tma_load_3d(sb + B_BYTES / 2, &tmB, full_bar(stage), k0, p.N + t.n0, 0);
            }
          } else {
            tma_load_3d(sb, &tmB, full_bar(stage), bk, t.b_n0, bg);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (so it can clean a ragged reduction tail in
    // shared memory); lane 0 alone issues the MMAs and commits.
    constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
    int stage = 0; uint32_t phase = 0;
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = !PAIR || leader;                      // the follower's MMA warp only allocates and frees tensor memory
    for (int tile = worker; tile < total_tiles && ok; tile += n_workers) {
      TileCoord t = get_tile(tile);
      if (!t.valid) continue;
      if (!mbar_wait(acce_bar(acc), acc_phase ^ 1u, 2, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
      uint32_t accumulate = 0;
      for (int k0 = t.k_lo; k0 < t.k_hi; k0 += BK) {
        if (!mbar_wait(full_bar(stage), phase, 3, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_base + stage * STAGE_BYTES, sb = sa + A_BYTES;
        if (A_MN && B_MN && p.group_mode == 2 && t.k_hi - k0 < BK) {
          // grouped reduction: rows past this group's end belong to the next group.
          // Zero them in the A tile (each k index is one 128-byte row per 64-wide box,
          // so whole-row zeroing is independent of the swizzle).
          const int valid = t.k_hi - k0;
          uint8_t* a_ptr = smem_al + stage * STAGE_BYTES;
          const int n16 = (BK - valid) * 8;                      // 16-byte pieces per box
          // A and B boxes are contiguous in the stage (2 + 4 boxes of 8 KB); B is cleared as well so that
          // a non-finite value in a foreign row cannot meet a zero
          for (int box = 0; box < (BM + BN) / 64; ++box)
            for (int i = lane; i < n16; i += 32)
              *reinterpret_cast<uint4*>(a_ptr + box * BOX_MN_BYTES + valid * 128 + i * 16) = make_uint4(0, 0, 0, 0);
          fence_proxy_async_smem();
        }
        __syncwarp();
        if (lane == 0) {
          // K-major: 16 bf16 = 32 B further along the 128 B row;
          // MN-major: 16 k-rows = two 8-row groups = 2048 B further.
          const uint64_t ad0 = A_MN ? umma_smem_desc(sa, BOX_MN_BYTES, 1024) : umma_smem_desc(sa, 16, 1024);
          const uint64_t bd0 = B_MN ? umma_smem_desc(sb, BOX_MN_BYTES, 1024) : umma_smem_desc(sb, 16, 1024);
          if (PAIR) {
            umma_bf16_pair(tmem_d, ad0, bd0, idesc, accumulate);
#pragma unroll
            for (int kk = 1; kk < BK / UMMA_K; ++kk)
              umma_bf16_pair(tmem_d, umma_desc_advance(ad0, kk * (A_MN ? 2048 : 32)), umma_desc_advance(bd0, kk * (B_MN ? 2048 : 32)), idesc, 1u);
            umma_commit_pair(empty_bar(stage));   // both CTAs' producers may refill the stage
          } else {
          umma_bf16(tmem_d, ad0, bd0, idesc, accumulate);
#pragma unroll
          for (int kk = 1; kk < BK / UMMA_K; ++kk)
            umma_bf16_acc(tmem_d, umma_desc_advance(ad0, kk * (A_MN ? 2048 : 32)), umma_desc_advance(bd0, kk * (B_MN ? 2048 : 32)), idesc);
          umma_commit(empty_bar(stage));          // stage reusable once these MMAs retire
          }
          accumulate = 1;
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (lane == 0) { if (PAIR) umma_commit_pair(accf_bar(acc)); else umma_commit(accf_bar(acc)); }  // accumulator complete
      __syncwarp();
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                        // TMEM lane quarter this warp may read
    int acc = 0; uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = worker; tile < total_tiles && ok; tile += n_workers) {
      TileCoord t = get_tile(tile);
      if (!t.valid) continue;
      if (EPI == EPI_SWIGLU_BWD) {
        // gate / up of the NEXT tile start moving into L2 now, a whole tile time before they are read
        auto prefetch_aux = [&](const TileCoord& tt) {
          const int prow = tt.m0 + q * 32 + lane, pcol = tt.n0 + ((warp - 2) >> 2) * (BN / 2);
          if (prow < tt.m_end) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int c = pcol + (i & 1) * 64;
              if (c < p.N)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(p.aux + (long long)prow * 2 * p.N + (i >> 1) * p.N + c));
            }
          }
        };
        if (tile == worker) prefetch_aux(t);
        const int nxt = tile + n_workers;
        if (nxt < total_tiles) { const TileCoord tn = get_tile(nxt); if (tn.valid) prefetch_aux(tn); }
      }
      if (!mbar_wait(accf_bar(acc), acc_phase, 4, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
      const int row = t.m0 + q * 32 + lane;
      const bool row_ok = row < t.m_end;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
      if (EPI == EPI_HEADS) {
        // One head (hd columns) at a time: TMEM -> RoPE -> bf16 -> swizzled staging tile(s) -> TMA store into
        // the head owner's packed tensor. The warp's 32 rows belong to one batch entry (rows_per_batch % 32 == 0).
        uint8_t* ebuf = smem_al + STAGES * STAGE_BYTES + (warp - 2) * 2 * EPI_BUF_BYTES;
        const uint32_t ebuf_s = smem_base + STAGES * STAGE_BYTES + (warp - 2) * 2 * EPI_BUF_BYTES;
        const int grow = t.m0 + q * 32;
        const bool rows_ok = grow < p.M;                       // warp-uniform (M % 32 == 0)
        const int bi = grow / p.rows_per_batch, t0 = grow - bi * p.rows_per_batch;
        const int hd = p.hd, half = hd >> 1;
        const int n_heads = p.Hq + 2 * p.Hkv;
        const uint4* csrow = reinterpret_cast<const uint4*>(p.cs + (long long)(t0 + lane) * hd);   // 4 (cos, sin) pairs per 16 bytes
        // rotate 32 (lo, hi) column pairs with their (cos, sin) entries: lo = columns [c, c+32), hi = [c+half, c+half+32)
        auto rotate = [&](uint32_t* lo, uint32_t* hi, const uint32_t* cs_lo, const uint32_t* cs_hi) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float2 l = __half22float2(*reinterpret_cast<const __half2*>(&cs_lo[i]));
            const float2 h = __half22float2(*reinterpret_cast<const __half2*>(&cs_hi[i]));
            const float a = __uint_as_float(lo[i]), b = __uint_as_float(hi[i]);
            lo[i] = __float_as_uint(a * l.x - b * l.y);
            hi[i] = __float_as_uint(b * h.x + a * h.y);
          }
        };
        auto load_cs = [&](uint32_t* dst, int c) {          // entries [c, c+32) of this row
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint4 v = csrow[(c >> 2) + i];
            dst[4 * i] = v.x; dst[4 * i + 1] = v.y; dst[4 * i + 2] = v.z; dst[4 * i + 3] = v.w;
          }
        };
        // 32 fp32 columns -> bf16 -> 16-byte chunks [chunk0, chunk0 + 4) of this lane's 128-byte staging row
        auto stage32 = [&](const uint32_t* r, uint8_t* buf, int chunk0) {
          uint8_t* rowp = buf + lane * 128;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            const int j = ch * 8;
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            v.y = pack_bf16(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            v.z = pack_bf16(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
            v.w = pack_bf16(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            *reinterpret_cast<uint4*>(rowp + (((chunk0 + ch) ^ (lane & 7)) << 4)) = v;
          }
        };
        const int heads_per_tile = BN / hd;
        uint32_t cs_lo[32], cs_hi[32];                       // hd 64: the row's whole table, shared by the tile's heads
        if (hd == 64 && rows_ok && t.n0 / hd < p.n_rot) { load_cs(cs_lo, 0); load_cs(cs_hi, 32); }
        if (hd == 32 && rows_ok && t.n0 / hd < p.n_rot) load_cs(cs_lo, 0);
#pragma unroll 1
        for (int hh = 0; hh < heads_per_tile; ++hh) {
          const int head = t.n0 / hd + hh;
          const bool live = rows_ok && head < n_heads;          // warp-uniform
          int dest, slot, copies = 1;
          if (head < p.Hq) { dest = head / p.q_l; slot = head - dest * p.q_l; }
          else if (p.kv_rep > 1) {                              // replicated KV heads: one local k and one local v slot
            const bool is_v = head >= p.Hq + p.Hkv;
            dest = (head - p.Hq - (is_v ? p.Hkv : 0)) * p.kv_rep; slot = p.q_l + (is_v ? 1 : 0); copies = p.kv_rep;
          }
          else if (head < p.Hq + p.Hkv) { const int k = head - p.Hq; dest = k / p.kv_l; slot = p.q_l + (k - dest * p.kv_l); }
          else { const int v = head - p.Hq - p.Hkv; dest = v / p.kv_l; slot = p.q_l + p.kv_l + (v - dest * p.kv_l); }
          const bool rot = head < p.n_rot;
          if (hd == 32) {
            // Heads of 32 columns: one TMEM load per head; the head fills the left half of a 64-column staging tile and
            // is stored with the same 64-wide box, whose right half lies outside the 32-wide head dimension of the
            // destination and is clipped by TMA.
            const int bsel = hh & 1;
            uint32_t r0[32];
            tmem_ld32(taddr + hh * 32, r0);
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
            tmem_ld_wait();
            if (live) {
              if (rot) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {                    // pairs (i, i + 16) with their own table entries
                  const float2 l = __half22float2(*reinterpret_cast<const __half2*>(&cs_lo[i]));
                  const float2 h = __half22float2(*reinterpret_cast<const __half2*>(&cs_lo[i + 16]));
                  const float a = __uint_as_float(r0[i]), b = __uint_as_float(r0[i + 16]);
                  r0[i] = __float_as_uint(a * l.x - b * l.y);
                  r0[i + 16] = __float_as_uint(b * h.x + a * h.y);
                }
              }
              stage32(r0, ebuf + bsel * EPI_BUF_BYTES, 0);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (live)
                for (int c = 0; c < copies; ++c)
                  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                               ::"l"((uint64_t)(dst_maps + dest + c)), "r"(ebuf_s + bsel * EPI_BUF_BYTES), "r"(0), "r"(slot),
                                 "r"(p.row_off + t0), "r"(bi) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          } else if (hd == 64) {
            const int bsel = hh & 1;
            uint32_t r0[32], r1[32];
            tmem_ld32(taddr + hh * 64, r0);
            tmem_ld32(taddr + hh * 64 + 32, r1);
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
            tmem_ld_wait();
            if (live) {
              if (rot) rotate(r0, r1, cs_lo, cs_hi);
              stage32(r0, ebuf + bsel * EPI_BUF_BYTES, 0);
              stage32(r1, ebuf + bsel * EPI_BUF_BYTES, 4);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (live)
                for (int c = 0; c < copies; ++c)
                  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                               ::"l"((uint64_t)(dst_maps + dest + c)), "r"(ebuf_s + bsel * EPI_BUF_BYTES), "r"(0), "r"(slot),
                                 "r"(p.row_off + t0), "r"(bi) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          } else {                                              // hd == 128: both staging tiles hold one head
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
#pragma unroll 1
            for (int part = 0; part < 2; ++part) {              // columns [32 part, +32) pair with [64 + 32 part, +32)
              uint32_t r0[32], r1[32];
              tmem_ld32(taddr + hh * 128 + part * 32, r0);
              tmem_ld32(taddr + hh * 128 + 64 + part * 32, r1);
              tmem_ld_wait();
              if (live) {
                if (rot) { load_cs(cs_lo, part * 32); load_cs(cs_hi, 64 + part * 32); rotate(r0, r1, cs_lo, cs_hi); }
                stage32(r0, ebuf, part * 4);
                stage32(r1, ebuf + EPI_BUF_BYTES, part * 4);
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (live) {
                for (int c = 0; c < copies; ++c)
#pragma unroll
                  for (int s2 = 0; s2 < 2; ++s2)
                    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                                 ::"l"((uint64_t)(dst_maps + dest + c)), "r"(ebuf_s + s2 * EPI_BUF_BYTES), "r"(s2 * 64), "r"(slot),
                                   "r"(p.row_off + t0), "r"(bi) : "memory");
              }
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        }
      } else if (EPI == EPI_SWIGLU || EPI == EPI_SWIGLU_BWD) {
        // forward: two 4 KB staging tiles per warp (4 warps); backward: one per warp (8 warps)
        constexpr int EBUF_PER_WARP = EPI == EPI_SWIGLU_BWD ? EPI_BUF_BYTES : 2 * EPI_BUF_BYTES;
        uint8_t* ebuf = smem_al + STAGES * STAGE_BYTES + (warp - 2) * EBUF_PER_WARP;
        const uint32_t ebuf_s = smem_base + STAGES * STAGE_BYTES + (warp - 2) * EBUF_PER_WARP;
        const int row0 = t.m0 + q * 32;
        int bsel = 0;
        // 64 bf16 columns (32 packed words) of this lane's row -> swizzled staging tile -> TMA store at (col, row0)
        // warps whose 32 rows all belong to the tile's row range use TMA tile stores; a warp that straddles the end
        // of its group (grouped mode) stores its rows one by one: `base` / `ld` locate the same tensor for that
        const bool whole = row0 + 32 <= t.m_end;               // warp-uniform
        auto put = [&](const uint32_t* w, const CUtensorMap* map, int col, __nv_bfloat16* base, long long ld) {
          if (!whole) {
            if (row0 + lane < t.m_end) {
              uint4* dst = reinterpret_cast<uint4*>(base + (long long)(row0 + lane) * ld + col);
#pragma unroll
              for (int ch = 0; ch < 8; ++ch) dst[ch] = make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
            }
            return;
          }
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          __syncwarp();
          uint8_t* rowp = ebuf + bsel * EPI_BUF_BYTES + lane * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(rowp + ((ch ^ (lane & 7)) << 4)) = make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (row0 < p.M)
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"((uint64_t)map), "r"(ebuf_s + bsel * EPI_BUF_BYTES), "r"(col), "r"(row0) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          bsel ^= 1;
        };
        if (EPI == EPI_SWIGLU) {
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {                      // two 64-column halves of the tile's 128 act columns
            uint32_t pg[32], pu[32], pa[32];
#pragma unroll
            for (int part = 0; part < 2; ++part) {
              uint32_t g[32], u[32];
              tmem_ld32(taddr + h * 64 + part * 32, g);
              tmem_ld32(taddr + 128 + h * 64 + part * 32, u);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const uint32_t gw = pack_bf16(__uint_as_float(g[i]), __uint_as_float(g[i + 1]));
                const uint32_t uw = pack_bf16(__uint_as_float(u[i]), __uint_as_float(u[i + 1]));
                const float2 gf = unpack_bf16(gw), uf = unpack_bf16(uw);
                pg[part * 16 + (i >> 1)] = gw;
                pu[part * 16 + (i >> 1)] = uw;
                pa[part * 16 + (i >> 1)] = pack_bf16(__fdividef(gf.x, 1.f + __expf(-gf.x)) * uf.x,
                                                     __fdividef(gf.y, 1.f + __expf(-gf.y)) * uf.y);
              }
            }
            const int col = t.n0 + h * 64;
            put(pg, &tmC, col, reinterpret_cast<__nv_bfloat16*>(p.C), p.ldc);
            put(pu, &tmC, p.N + col, reinterpret_cast<__nv_bfloat16*>(p.C), p.ldc);
            put(pa, dst_maps, col, p.act, p.ld_act);
          }
        } else {
          // d(act) leaves tensor memory one row per lane, but the derivative is elementwise, so the warp stages
          // the bf16 tile in shared memory and re-reads it with 8 lanes per row: gate / up then come from global
          // memory as whole 128-byte rows (4 rows per load instruction instead of 32 scattered pieces) and the
          // results go back the same way.
          uint8_t* buf = ebuf;
          const int sub_row = lane >> 3, chunk = lane & 7;    // this lane's (row within a group of 4, 16-byte chunk)
          const int slab0 = ((warp - 2) >> 2) * (BN / 128);    // this warp's half of the tile's four 64-column slabs
#pragma unroll 1
          for (int slab = slab0; slab < slab0 + BN / 128; ++slab) {
            const int col = t.n0 + slab * 64;
            if (col >= p.N) break;                             // warp-uniform
            uint32_t d0[32], d1[32];
            tmem_ld32(taddr + slab * 64, d0);
            tmem_ld32(taddr + slab * 64 + 32, d1);
            tmem_ld_wait();
            {
              uint8_t* rowp = buf + lane * 128;
#pragma unroll
              for (int ch = 0; ch < 8; ++ch) {
                const uint32_t* r = ch < 4 ? d0 : d1;
                const int j = (ch & 3) * 8;
                uint4 v;
                v.x = pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                v.y = pack_bf16(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                v.z = pack_bf16(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                v.w = pack_bf16(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                *reinterpret_cast<uint4*>(rowp + ((ch ^ (lane & 7)) << 4)) = v;
              }
            }
            // all of this slab's gate / up loads are issued before the first store (the compiler must assume the
            // stores may alias them, so it would not hoist them itself); they overlap the staging above
            uint4 gv[8], uv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int grow = row0 + i * 4 + sub_row;
              gv[i] = make_uint4(0, 0, 0, 0); uv[i] = gv[i];
              if (grow < t.m_end && col + chunk * 8 < p.N) {
                const __nv_bfloat16* gp = p.aux + (long long)grow * 2 * p.N + col + chunk * 8;
                gv[i] = *reinterpret_cast<const uint4*>(gp);
                uv[i] = *reinterpret_cast<const uint4*>(gp + p.N);
              }
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + sub_row;                   // row within the warp's 32
              const int grow = row0 + r;
              const uint32_t off = r * 128 + ((chunk ^ (r & 7)) << 4);
              const bool live = grow < t.m_end && col + chunk * 8 < p.N;
              const uint4 dv = *reinterpret_cast<const uint4*>(buf + off);
              const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w}, gw[4] = {gv[i].x, gv[i].y, gv[i].z, gv[i].w},
                             uw[4] = {uv[i].x, uv[i].y, uv[i].z, uv[i].w};
              uint32_t og[4], ou[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float2 dd = unpack_bf16(dw[k]), a = unpack_bf16(gw[k]), bb = unpack_bf16(uw[k]);
                const float s0 = __fdividef(1.f, 1.f + __expf(-a.x)), s1 = __fdividef(1.f, 1.f + __expf(-a.y));
                og[k] = pack_bf16(dd.x * bb.x * s0 * (1.f + a.x * (1.f - s0)), dd.y * bb.y * s1 * (1.f + a.y * (1.f - s1)));
                ou[k] = pack_bf16(dd.x * a.x * s0, dd.y * a.y * s1);
              }
              if (live) {                                      // 8 lanes write one 128-byte row piece of d(gate) and of d(up)
                __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)grow * p.ldc + col + chunk * 8;
                *reinterpret_cast<uint4*>(op) = make_uint4(og[0], og[1], og[2], og[3]);
                *reinterpret_cast<uint4*>(op + p.N) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
              }
            }
            __syncwarp();
          }
        }
      } else if (EPI == EPI_LSE) {
        // this thread's row of the tile: running maximum and sum of exponentials over 256 columns, 32 at a time
        const long long tgt = row_ok ? p.targets[row] : -1;
        float m_run = -INFINITY, s_run = 0.f;
        constexpr float LOG2E = 1.4426950408889634f;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c, r);
          tmem_ld_wait();
          const int col = t.n0 + c;
          if (col >= p.N) break;                                  // warp-uniform
          float v[32];
          float cmax = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; j += 2) {                       // logits as the bf16 values a stored tile would hold
            const float2 f = unpack_bf16(pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1])));
            v[j] = col + j < p.N ? f.x : -INFINITY;
            v[j + 1] = col + j + 1 < p.N ? f.y : -INFINITY;
            cmax = fmaxf(cmax, fmaxf(v[j], v[j + 1]));
          }
          if (tgt >= col && tgt < col + 32) {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (tgt == col + j) p.tgt_logit[row] = v[j];
          }
          const float m_new = fmaxf(m_run, cmax);
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) acc += ex2_approx((v[j] - m_new) * LOG2E);
          s_run = s_run * ex2_approx((m_run - m_new) * LOG2E) + acc;
          m_run = m_new;
        }
        if (row_ok) p.lse_part[(long long)row * p.lse_tiles + t.n0 / BN] = make_float2(m_run, s_run);
      } else if (EPI == EPI_BF16 && p.tma_store) {
        // 64-column slabs: TMEM -> bf16 -> swizzled staging tile -> TMA store (clips at the matrix edge).
        uint8_t* ebuf = smem_al + STAGES * STAGE_BYTES + (warp - 2) * 2 * EPI_BUF_BYTES;
        const uint32_t ebuf_s = smem_base + STAGES * STAGE_BYTES + (warp - 2) * 2 * EPI_BUF_BYTES;
#pragma unroll 1
        for (int slab = 0; slab < BN / 64; ++slab) {
          const int bsel = slab & 1;
          uint32_t r0[32], r1[32];
          tmem_ld32(taddr + slab * 64, r0);
          tmem_ld32(taddr + slab * 64 + 32, r1);
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // this buffer's previous store has read it
          __syncwarp();
          tmem_ld_wait();
          if (p.dl_lse != nullptr) {
            constexpr float LOG2E = 1.4426950408889634f;
            const long long tg = row_ok ? p.targets[row] : p.dl_ignore;
            const float sc = tg != p.dl_ignore ? *p.dl_scale : 0.f;
            const float nl = row_ok ? -p.dl_lse[row] * LOG2E : 0.f;
            const int col0 = t.n0 + slab * 64;
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float2 a = unpack_bf16(pack_bf16(__uint_as_float(r0[j]), __uint_as_float(r0[j + 1])));
              const float2 b = unpack_bf16(pack_bf16(__uint_as_float(r1[j]), __uint_as_float(r1[j + 1])));
              float pa0 = ex2_approx(fmaf(a.x, LOG2E, nl)), pa1 = ex2_approx(fmaf(a.y, LOG2E, nl));
              float pb0 = ex2_approx(fmaf(b.x, LOG2E, nl)), pb1 = ex2_approx(fmaf(b.y, LOG2E, nl));
              if (tg == col0 + j) pa0 -= 1.f;
              if (tg == col0 + j + 1) pa1 -= 1.f;
              if (tg == col0 + 32 + j) pb0 -= 1.f;
              if (tg == col0 + 32 + j + 1) pb1 -= 1.f;
              r0[j] = __float_as_uint(pa0 * sc); r0[j + 1] = __float_as_uint(pa1 * sc);
              r1[j] = __float_as_uint(pb0 * sc); r1[j + 1] = __float_as_uint(pb1 * sc);
            }
          }
          uint8_t* rowp = ebuf + bsel * EPI_BUF_BYTES + lane * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint32_t* r = ch < 4 ? r0 : r1;
            const int j = (ch & 3) * 8;
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            v.y = pack_bf16(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            v.z = pack_bf16(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
            v.w = pack_bf16(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            *reinterpret_cast<uint4*>(rowp + ((ch ^ (lane & 7)) << 4)) = v;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int c0 = t.n0 + slab * 64, c1 = t.m0 + q * 32;
            if (c0 < p.N && c1 < p.M)
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"((uint64_t)&tmC), "r"(ebuf_s + bsel * EPI_BUF_BYTES), "r"(c0), "r"(c1) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      } else if (EPI == EPI_F32_ACC && p.tma_store) {
        // C += accumulator through TMA reduce-add: 32-column fp32 slabs are staged (swizzled) in shared memory and added
        // to C in L2 as whole 128-byte rows. No C value travels to the SM, nothing waits on a global load, and a
        // split reduction's partial sums meet in L2 the same way (their order is then not fixed; an unsplit GEMM adds
        // exactly one value to each element and stays deterministic).
        uint8_t* ebuf = smem_al + STAGES * STAGE_BYTES + (warp - 2) * 2 * EPI_BUF_BYTES;
        const uint32_t ebuf_s = smem_base + STAGES * STAGE_BYTES + (warp - 2) * 2 * EPI_BUF_BYTES;
        const int row0 = t.m0 + q * 32;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          const int bsel = (c >> 5) & 1;
          uint32_t r[32];
          tmem_ld32(taddr + c, r);
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // this buffer's previous reduce has read it
          __syncwarp();
          tmem_ld_wait();
          uint8_t* rowp = ebuf + bsel * EPI_BUF_BYTES + lane * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(rowp + ((ch ^ (lane & 7)) << 4)) = make_uint4(r[4 * ch], r[4 * ch + 1], r[4 * ch + 2], r[4 * ch + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (t.n0 + c < p.N && row0 < p.M)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                           ::"l"((uint64_t)&tmC), "r"(ebuf_s + bsel * EPI_BUF_BYTES), "r"(t.n0 + c), "r"(row0) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      } else if (EPI == EPI_ROWS) {
        // Each output row goes to a looked-up (buffer, row), usually in another GPU's memory. The accumulator leaves
        // tensor memory one row per lane; stored that way every store instruction would write 32 separate 16-byte
        // pieces, a poor packet size for NVLink. So each 64-column slab is staged in shared memory (swizzled, one
        // 128-byte row per lane) and written back with 8 lanes per row: one instruction stores four whole 128-byte
        // row pieces. The lane that owns a row holds its destination; the writers fetch it with shuffles.
        uint8_t* buf = smem_al + STAGES * STAGE_BYTES + (warp - 2) * 2 * EPI_BUF_BYTES;
        unsigned long long dst_bits = 0;               // 0: the row is dropped
        {
          const int dr = row_ok ? p.rs_rank[row] : -1;
          const long long drow = dr >= 0 ? p.rs_row[row] : -1;
          if (dr >= 0 && dr < MAX_HEAD_DST && drow >= 0 && drow < p.rs_rows)
            dst_bits = reinterpret_cast<unsigned long long>(reinterpret_cast<__nv_bfloat16*>(p.rs_dst[dr]) + drow * p.ldc);
          else if (dr >= 0)
            report_status(p.status, (61u << 8) | 1u);
        }
        const int sub_row = lane >> 3, chunk = lane & 7;
#pragma unroll 1
        for (int slab = 0; slab < BN / 64; ++slab) {
          const int col = t.n0 + slab * 64;
          if (col >= p.N) break;                               // warp-uniform
          uint32_t r0[32], r1[32];
          tmem_ld32(taddr + slab * 64, r0);
          tmem_ld32(taddr + slab * 64 + 32, r1);
          tmem_ld_wait();
          uint8_t* rowp = buf + lane * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint32_t* r = ch < 4 ? r0 : r1;
            const int j = (ch & 3) * 8;
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            v.y = pack_bf16(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            v.z = pack_bf16(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
            v.w = pack_bf16(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            *reinterpret_cast<uint4*>(rowp + ((ch ^ (lane & 7)) << 4)) = v;
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + sub_row;                     // row within the warp's 32
            const unsigned long long d = __shfl_sync(0xffffffffu, dst_bits, r);
            const uint4 v = *reinterpret_cast<const uint4*>(buf + r * 128 + ((chunk ^ (r & 7)) << 4));
            if (d != 0 && col + chunk * 8 < p.N)
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(d) + col + chunk * 8) = v;
          }
          __syncwarp();
        }
      } else {
      const bool row_live = row_ok;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c, r);
        tmem_ld_wait();
        const int col = t.n0 + c;
        if (row_live && col < p.N) {
          if (EPI == EPI_BF16) {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + t.c_off + (long long)row * p.ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col + j < p.N) {
                uint4 v;
                v.x = pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                v.y = pack_bf16(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                v.z = pack_bf16(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                v.w = pack_bf16(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                *reinterpret_cast<uint4*>(out + j) = v;
              }
            }
          } else {
            float* out = reinterpret_cast<float*>(p.C) + t.c_off + (long long)row * p.ldc + col;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col + j < p.N) {
                float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                       __uint_as_float(r[j + 3]));
                if (EPI == EPI_F32_ACC && p.split_k > 1) {
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + j), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
                } else {
                  if (EPI == EPI_F32_ACC) {
                    const float4 o = *reinterpret_cast<const float4*>(out + j);
                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                  }
                  *reinterpret_cast<float4*>(out + j) = v;
                }
              }
            }
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && !leader) mbar_arrive_cluster(mapa_shared(acce_bar(acc), 0));
        else mbar_arrive(acce_bar(acc));
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if ((((EPI == EPI_BF16 || EPI == EPI_F32_ACC) && p.tma_store) || EPI == EPI_HEADS || EPI == EPI_SWIGLU || EPI == EPI_SWIGLU_BWD) && lane == 0)
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  if (PAIR) cluster_sync_all();          // neither CTA leaves (or frees tensor memory) while its peer may still signal or read it
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, int EPI, bool GATED = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  gemm_body<A_MN, B_MN, EPI, GATED>(tmA, tmB, tmC, p, nullptr);
}

// Same main loop, head-scatter epilogue: the output maps (one per destination rank) replace the C map.
template <bool B_MN, bool GATED = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_heads_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ HeadDstMaps dst, const GemmParams p) {
  gemm_body<false, B_MN, EPI_HEADS, GATED>(tmA, tmB, tmA, p, dst.m);
}

// MLP forward / backward with the SwiGLU math in the epilogue: `tmC` is the [M, 2 I] tensor the epilogue
// stores gate|up (forward) or d(gate)|d(up) (backward) into, `tmD` the forward's act [M, I].
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_swiglu_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmD, const GemmParams p) {
  gemm_body<false, false, EPI_SWIGLU>(tmA, tmB, tmC, p, &tmD);
}
__global__ void __launch_bounds__(GEMM_THREADS_WIDE, 1)
gemm_swiglu_bwd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  gemm_body<false, true, EPI_SWIGLU_BWD>(tmA, tmB, tmC, p, nullptr);
}

// CTA-pair instantiations (clusters of two CTAs, see gemm_body): plain GEMMs and the dense fused epilogues.
template <bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  gemm_body<A_MN, B_MN, EPI, false, true>(tmA, tmB, tmC, p, nullptr);
}
template <bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_heads_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ HeadDstMaps dst, const GemmParams p) {
  gemm_body<false, B_MN, EPI_HEADS, false, true>(tmA, tmB, tmA, p, dst.m);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_swiglu_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmD,
                        const GemmParams p) {
  gemm_body<false, false, EPI_SWIGLU, false, true>(tmA, tmB, tmC, p, &tmD);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS_WIDE, 1)
gemm_swiglu_bwd_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                            const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  gemm_body<false, true, EPI_SWIGLU_BWD, false, true>(tmA, tmB, tmC, p, nullptr);
}

// ---- host side ---------------------------------------------------------------------------------
// CTA pairs are used for every plain (ungrouped, ungated) GEMM of at least 256 rows unless switched off
// (TLM_GEMM_PAIR=0 in the environment, or tlm_gemm_set_pair).
static int g_pair_mode = -1;
static bool pair_enabled() {
  if (g_pair_mode < 0) {
    const char* e = getenv("TLM_GEMM_PAIR");
    g_pair_mode = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return g_pair_mode != 0;
}
static bool use_pair(int M) { return pair_enabled() && M >= 2 * BM && num_sms() >= 2; }
// row-grouped GEMMs: a pair tile's second half is wasted at the end of every group, so pairs need large groups
// (mode 2, set by tests: pairs for every row-grouped launch, so that small ragged groups exercise that path)
static bool use_pair_grouped(int M, int groups) { return use_pair(M) && (g_pair_mode == 2 || (long long)M >= 512LL * groups); }
// grid of a pair kernel: two CTAs per tile walker, at most one walker per SM pair
static int pair_grid(long long tiles) {
  const int walkers = num_sms() / 2;
  return 2 * (int)(tiles < walkers ? tiles : walkers);
}
// Operand description: `ptr` points at element (0,0); K-major operands are
// [rows, K] with leading dimension `ld`; MN-major operands are [K, rows] with
// leading dimension `ld`. `groups`/`group_stride` add an outer dimension (B only).
struct Operand {
  const void* ptr;
  long long rows, k, ld;
  bool mn_major;
  long long groups, group_stride;
};

static int build_map(CUtensorMap* map, const Operand& o, int box_rows) {
  uint64_t dims[3], strides[2];
  uint32_t box[3];
  if (o.mn_major) {            // memory [k][rows]: inner = rows
    dims[0] = (uint64_t)o.rows; dims[1] = (uint64_t)o.k;
    box[0] = 64; box[1] = BK;
  } else {                     // memory [rows][k]: inner = k
    dims[0] = (uint64_t)o.k; dims[1] = (uint64_t)o.rows;
    box[0] = BK; box[1] = (uint32_t)box_rows;
  }
  strides[0] = (uint64_t)o.ld * 2;
  int rank = 2;
  if (o.groups > 0) {
    dims[2] = (uint64_t)o.groups; strides[1] = (uint64_t)o.group_stride * 2; box[2] = 1; rank = 3;
  }
  return make_tmap_bf16(map, o.ptr, rank, dims, strides, box);
}

template <bool A_MN, bool B_MN, int EPI, bool GATED = false>
static int launch_t(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const GemmParams& p, int tiles,
                    cudaStream_t st) {
  static bool configured = false;
  auto kern = gemm_kernel<A_MN, B_MN, EPI, GATED>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int grid = tiles < num_sms() ? tiles : num_sms();
  if (grid <= 0) return 0;
  kern<<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(ma, mb, mc, p);
  count_launch();
  return launch_status();
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_pair_t(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const GemmParams& p,
                         int tiles, cudaStream_t st) {
  static bool configured = false;
  auto kern = gemm_pair_kernel<A_MN, B_MN, EPI>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_PAIR);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int grid = pair_grid(tiles);
  if (grid <= 0) return 0;
  kern<<<grid, GEMM_THREADS, GEMM_SMEM_PAIR, st>>>(ma, mb, mc, p);
  count_launch();
  return launch_status();
}

// `pair`: `tiles` counts 256-row tiles and the B map was built with 128-row boxes (see pair_maps)
static int dispatch(bool a_mn, bool b_mn, int epi, const CUtensorMap& ma, const CUtensorMap& mb, GemmParams p,
                    int tiles, cudaStream_t st, bool pair = false) {
  CUtensorMap mc = ma;                      // placeholder when the TMA-store epilogue is off
  if (p.split_k < 1) { p.split_k = 1; p.k_chunk = p.K; }
  if (epi == EPI_BF16 && p.groups == 0 && p.ldc % 8 == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0) {
    uint64_t dims[2] = {(uint64_t)p.N, (uint64_t)p.M}, strides[1] = {(uint64_t)p.ldc * 2};
    uint32_t box[2] = {64, 32};
    if (make_tmap_bf16(&mc, p.C, 2, dims, strides, box) == 0) p.tma_store = 1;
  }
  static int f32_reduce = -1;                 // TLM_GEMM_TMA_REDUCE=0: fp32 accumulation with loads and stores / red.global
  if (f32_reduce < 0) { const char* v = getenv("TLM_GEMM_TMA_REDUCE"); f32_reduce = (v != nullptr && v[0] == '0') ? 0 : 1; }
  if (epi == EPI_F32_ACC && f32_reduce && p.groups == 0 && p.ldc % 4 == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0) {
    uint64_t dims[2] = {(uint64_t)p.N, (uint64_t)p.M}, strides[1] = {(uint64_t)p.ldc * 4};
    uint32_t box[2] = {32, 32};
    if (make_tmap_f32(&mc, p.C, 2, dims, strides, box) == 0) p.tma_store = 1;
  }
  if (p.dl_lse != nullptr && !p.tma_store) return -6;       // the gradient transform lives in the TMA-store epilogue
  // x W^T with a pending "parameters ready" gate: the gated instantiation (see gemm_body)
  if (!a_mn && !b_mn && epi == EPI_BF16 && p.wait_flags[0] != nullptr)
    return launch_t<false, false, EPI_BF16, true>(ma, mb, mc, p, tiles, st);
  if (pair && ((p.groups != 0 && p.group_mode != 1) || p.wait_flags[0] != nullptr)) return -8;
#define TLM_CASE(A, B, E)                                                          \
  if (a_mn == A && b_mn == B && epi == E)                                          \
    return pair ? launch_pair_t<A, B, E>(ma, mb, mc, p, tiles, st) : launch_t<A, B, E>(ma, mb, mc, p, tiles, st);
  TLM_CASE(false, false, EPI_BF16) TLM_CASE(false, true, EPI_BF16) TLM_CASE(true, true, EPI_F32_ACC)
  TLM_CASE(false, false, EPI_F32) TLM_CASE(true, true, EPI_F32) TLM_CASE(false, false, EPI_F32_ACC)
  TLM_CASE(true, true, EPI_BF16) TLM_CASE(false, true, EPI_F32) TLM_CASE(false, false, EPI_LSE)
  TLM_CASE(false, false, EPI_ROWS) TLM_CASE(false, true, EPI_ROWS)
#undef TLM_CASE
  return -2;
}

template <bool B_MN, bool GATED = false>
static int launch_heads(const CUtensorMap& ma, const CUtensorMap& mb, const HeadDstMaps& dst, const GemmParams& p,
                        int tiles, cudaStream_t st) {
  static bool configured = false;
  auto kern = gemm_heads_kernel<B_MN, GATED>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int grid = tiles < num_sms() ? tiles : num_sms();
  if (grid <= 0) return 0;
  kern<<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(ma, mb, dst, p);
  count_launch();
  return launch_status();
}

template <bool B_MN>
static int launch_heads_pair(const CUtensorMap& ma, const CUtensorMap& mb, const HeadDstMaps& dst, const GemmParams& p,
                             int tiles, cudaStream_t st) {
  static bool configured = false;
  auto kern = gemm_heads_pair_kernel<B_MN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_PAIR);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int grid = pair_grid(tiles);
  if (grid <= 0) return 0;
  kern<<<grid, GEMM_THREADS, GEMM_SMEM_PAIR, st>>>(ma, mb, dst, p);
  count_launch();
  return launch_status();
}

}  // namespace tlm

using namespace tlm;

// CTA-pair GEMMs at run time (tests and A/B measurements): 0 off, 1 on, 2 on and also for row-grouped GEMMs with
// small groups. Returns the previous setting.
TLM_API int tlm_gemm_set_pair(int mode) {
  pair_enabled();
  const int was = g_pair_mode;
  g_pair_mode = mode < 0 ? 0 : (mode > 2 ? 2 : mode);
  return was;
}

// Projection GEMM whose epilogue applies RoPE and scatters heads (see GemmParams):
//   A [M = batch * rows_per_batch, K] (lda);  B [N, K] K-major (b_mn = 0) or [K, N] MN-major (b_mn = 1),
//   N = (Hq + 2 Hkv) * hd;  dst_ptrs[r]: bf16 [batch, dst_rows, dst_heads, hd] on rank r (peer-mapped
//   addresses are fine: the stores are TMA tile stores without multicast);  cs: fp16 (cos, sin) pairs
//   [rows_per_batch, hd, 2] for the heads below n_rot.
// Requirements: hd in {32, 64, 128}, rows_per_batch % 32 == 0, n_dst <= 8, Hq % q_l == 0, Hkv % kv_l == 0.
TLM_API int tlm_gemm_heads(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, int b_mn,
                           void* const* dst_ptrs, int n_dst, int batch, int rows_per_batch, int dst_rows, int dst_heads,
                           int row_off, int Hq, int Hkv, int q_l, int kv_l, int hd, int n_rot, const void* cs,
                           int kv_rep, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((hd != 32 && hd != 64 && hd != 128) || rows_per_batch % 32 != 0 || n_dst < 1 || n_dst > MAX_HEAD_DST) return -4;
  if (M != batch * rows_per_batch || N != (Hq + 2 * Hkv) * hd || q_l <= 0 || Hq % q_l != 0) return -5;
  if (kv_rep < 1) kv_rep = 1;
  if (kv_rep > 1) {                     // replicated KV heads: every destination holds exactly one k and one v head
    if (Hkv <= 0 || Hkv * kv_rep > n_dst || Hq / q_l > n_dst) return -5;
    kv_l = 1;
  } else {
    if (Hkv > 0 && (kv_l <= 0 || Hkv % kv_l != 0)) return -5;
    if (Hq / q_l > n_dst || (Hkv > 0 && Hkv / kv_l > n_dst)) return -5;
  }
  if (n_rot > 0 && cs == nullptr) return -5;
  GemmParams p{};
  if (!b_mn) take_pending_waits(p);               // x W^T: may be the first reader of its weights after an optimizer step
  const bool pair = use_pair(M) && p.wait_flags[0] == nullptr;
  Operand oa{A, M, K, lda, false, 0, 0}, ob{B, N, K, ldb, b_mn != 0, 1, (long long)N * K};
  CUtensorMap ma, mb;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  e = build_map(&mb, ob, pair ? BN / 2 : BN);
  if (e) return e;
  HeadDstMaps dst;
  for (int r = 0; r < n_dst; ++r) {
    e = make_qkv_map(&dst.m[r], dst_ptrs[r], batch, dst_rows, dst_heads, hd, 32);
    if (e) return e;
  }
  for (int r = n_dst; r < MAX_HEAD_DST; ++r) dst.m[r] = dst.m[0];
  p.M = M; p.N = N; p.K = K; p.C = nullptr; p.ldc = 0; p.status = status_word(); p.groups = 0;
  p.split_k = 1; p.k_chunk = K;
  p.hd = hd; p.rows_per_batch = rows_per_batch; p.row_off = row_off; p.Hq = Hq; p.Hkv = Hkv;
  p.q_l = q_l; p.kv_l = kv_l > 0 ? kv_l : 1; p.n_rot = n_rot; p.cs = (const __half2*)cs; p.kv_rep = kv_rep;
  if (pair) {
    const int ptiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    return b_mn ? launch_heads_pair<true>(ma, mb, dst, p, ptiles, stream) : launch_heads_pair<false>(ma, mb, dst, p, ptiles, stream);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if (!b_mn && p.wait_flags[0] != nullptr) return launch_heads<false, true>(ma, mb, dst, p, tiles, stream);
  return b_mn ? launch_heads<true>(ma, mb, dst, p, tiles, stream) : launch_heads<false>(ma, mb, dst, p, tiles, stream);
}

static int store_map_bf16(CUtensorMap* m, void* base, long long rows, long long cols, long long ld) {
  uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows}, strides[1] = {(uint64_t)ld * 2};
  uint32_t box[2] = {64, 32};
  return make_tmap_bf16(m, base, 2, dims, strides, box);
}

// gate_up[M, 2 I] = x[M, K] * w_gu[2 I, K]^T  and  act[M, I] = silu(gate) * up, in one kernel.
// Requirements: I % 128 == 0, contiguous outputs (row pitches 2 I and I).
TLM_API int tlm_gemm_swiglu(const void* x, const void* w_gu, void* gate_up, void* act, int M, int I, int K,
                            long long lda, long long ldb, cudaStream_t stream) {
  if (M <= 0 || I <= 0 || K <= 0) return 0;
  if (I % 128 != 0) return -4;
  Operand oa{x, M, K, lda, false, 0, 0}, ob{w_gu, 2LL * I, K, ldb, false, 1, 2LL * I * K};
  CUtensorMap ma, mb, mc, md;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  e = build_map(&mb, ob, 128);
  if (e) return e;
  e = store_map_bf16(&mc, gate_up, M, 2LL * I, 2LL * I);
  if (e) return e;
  e = store_map_bf16(&md, act, M, I, I);
  if (e) return e;
  GemmParams p{};
  p.M = M; p.N = I; p.K = K; p.C = gate_up; p.ldc = 2LL * I; p.status = status_word(); p.split_k = 1; p.k_chunk = K;
  p.act = (__nv_bfloat16*)act; p.ld_act = I;
  if (use_pair(M)) {               // the B map's 128-row boxes serve both forms: rank 0 loads gate rows, rank 1 up rows
    static bool pconfigured = false;
    if (!pconfigured) {
      cudaError_t ce = cudaFuncSetAttribute(gemm_swiglu_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_PAIR);
      if (ce != cudaSuccess) return (int)ce;
      pconfigured = true;
    }
    const int pgrid = pair_grid((long long)((M + 2 * BM - 1) / (2 * BM)) * (I / 128));
    gemm_swiglu_pair_kernel<<<pgrid, GEMM_THREADS, GEMM_SMEM_PAIR, stream>>>(ma, mb, mc, md, p);
    count_launch();
    return launch_status();
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_swiglu_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * (I / 128);
  const int grid = tiles < num_sms() ? tiles : num_sms();
  gemm_swiglu_kernel<<<grid, GEMM_THREADS, GEMM_SMEM, stream>>>(ma, mb, mc, md, p);
  count_launch();
  return launch_status();
}

// d(gate_up)[M, 2 I] from dy[M, D], w_down[D, I] (row pitch ldb) and the saved gate_up[M, 2 I]:
// d(act) = dy * w_down never reaches memory, the epilogue applies the SwiGLU derivative.
TLM_API int tlm_gemm_swiglu_bwd(const void* dy, const void* w_down, const void* gate_up, void* d_gate_up, int M, int I,
                                int D, long long lda, long long ldb, cudaStream_t stream) {
  if (M <= 0 || I <= 0 || D <= 0) return 0;
  if (I % 8 != 0) return -4;
  Operand oa{dy, M, D, lda, false, 0, 0}, ob{w_down, I, D, ldb, true, 1, (long long)I * D};
  CUtensorMap ma, mb, mc;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  e = build_map(&mb, ob, BN);
  if (e) return e;
  e = store_map_bf16(&mc, d_gate_up, M, 2LL * I, 2LL * I);
  if (e) return e;
  GemmParams p{};
  p.M = M; p.N = I; p.K = D; p.C = d_gate_up; p.ldc = 2LL * I; p.status = status_word(); p.split_k = 1; p.k_chunk = D;
  p.aux = (const __nv_bfloat16*)gate_up;
  if (use_pair(M)) {               // MN-major B: 64-wide boxes in both forms
    static bool pconfigured = false;
    if (!pconfigured) {
      cudaError_t ce = cudaFuncSetAttribute(gemm_swiglu_bwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_PAIR);
      if (ce != cudaSuccess) return (int)ce;
      pconfigured = true;
    }
    const int pgrid = pair_grid((long long)((M + 2 * BM - 1) / (2 * BM)) * ((I + BN - 1) / BN));
    gemm_swiglu_bwd_pair_kernel<<<pgrid, GEMM_THREADS_WIDE, GEMM_SMEM_PAIR, stream>>>(ma, mb, mc, p);
    count_launch();
    return launch_status();
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_swiglu_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((I + BN - 1) / BN);
  const int grid = tiles < num_sms() ? tiles : num_sms();
  gemm_swiglu_bwd_kernel<<<grid, GEMM_THREADS_WIDE, GEMM_SMEM, stream>>>(ma, mb, mc, p);
  count_launch();
  return launch_status();
}

// Arms a "parameters ready" gate for the next forward-projection GEMM launched through this library (tlm_gemm with
// x W^T and a bf16 result, or tlm_gemm_heads): its producer warp waits until all `n` ranks' updates of `bucket` have
// arrived (`ready_local`: this rank's READY_INTS-word flag array in symmetric memory). Up to two gates can be pending;
// the launch that takes them clears them. Other GEMM entry points leave pending gates alone;
// tlm_gemm_flush_param_waits turns gates that nobody took into stand-alone wait kernels.
TLM_API int tlm_gemm_arm_param_wait(const int* ready_local, int bucket, int n) {
  if (ready_local == nullptr || bucket < 0 || bucket >= READY_MAX_BUCKETS || n < 1 || n > READY_STRIDE) return -6;
  if (g_n_pending_wait >= 2) return -7;
  g_pending_wait[g_n_pending_wait].flags = ready_local;
  g_pending_wait[g_n_pending_wait].bucket = bucket;
  g_pending_wait[g_n_pending_wait].n = n;
  ++g_n_pending_wait;
  return 0;
}
TLM_API void tlm_gemm_clear_param_waits() { g_n_pending_wait = 0; }
TLM_API int tlm_wait_params_ready(const int* ready_local, int bucket, int n, cudaStream_t st);
// Queue every pending gate as a one-warp wait kernel on `stream` (the gates' GEMM never came) and clear them.
TLM_API int tlm_gemm_flush_param_waits(cudaStream_t stream) {
  int rc = 0;
  for (int i = 0; i < g_n_pending_wait && rc == 0; ++i)
    rc = tlm_wait_params_ready(g_pending_wait[i].flags, g_pending_wait[i].bucket, g_pending_wait[i].n, stream);
  g_n_pending_wait = 0;
  return rc;
}

// MoE experts, forward: rows of x [R, K] are grouped by expert (`row_start`, device, groups + 1 ints); group g gets
//   gate_up[rows_g] = x[rows_g] * [W_g ; W_{groups+g}]^T   (W: 2 * groups matrices [I, K], `w_group_stride` apart)
//   act[rows_g]     = silu(gate) * up
// in one kernel (the dense MLP's SwiGLU epilogue with the expert picked per tile). I % 128 == 0.
TLM_API int tlm_gemm_swiglu_grouped(const void* x, const void* w_pair, void* gate_up, void* act, const int* row_start,
                                    int groups, int R, int I, int K, long long lda, long long w_group_stride,
                                    int max_rows_per_group, cudaStream_t stream) {
  if (R <= 0 || I <= 0 || K <= 0 || groups <= 0) return 0;
  if (I % 128 != 0) return -4;
  Operand oa{x, R, K, lda, false, 0, 0}, ob{w_pair, I, K, K, false, 2LL * groups, w_group_stride};
  CUtensorMap ma, mb, mc, md;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  e = build_map(&mb, ob, 128);
  if (e) return e;
  e = store_map_bf16(&mc, gate_up, R, 2LL * I, 2LL * I);
  if (e) return e;
  e = store_map_bf16(&md, act, R, I, I);
  if (e) return e;
  GemmParams p{};
  p.M = R; p.N = I; p.K = K; p.C = gate_up; p.ldc = 2LL * I; p.status = status_word(); p.split_k = 1; p.k_chunk = K;
  p.act = (__nv_bfloat16*)act; p.ld_act = I;
  p.groups = groups; p.row_start = row_start; p.group_mode = 1;
  if (use_pair_grouped(R, groups)) {
    p.max_tiles_m = (max_rows_per_group + 2 * BM - 1) / (2 * BM);
    static bool pconfigured = false;
    if (!pconfigured) {
      cudaError_t ce = cudaFuncSetAttribute(gemm_swiglu_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_PAIR);
      if (ce != cudaSuccess) return (int)ce;
      pconfigured = true;
    }
    const int pgrid = pair_grid((long long)groups * p.max_tiles_m * (I / 128));
    gemm_swiglu_pair_kernel<<<pgrid, GEMM_THREADS, GEMM_SMEM_PAIR, stream>>>(ma, mb, mc, md, p);
    count_launch();
    return launch_status();
  }
  p.max_tiles_m = (max_rows_per_group + BM - 1) / BM;
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_swiglu_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  const int tiles = groups * p.max_tiles_m * (I / 128);
  const int grid = tiles < num_sms() ? tiles : num_sms();
  gemm_swiglu_kernel<<<grid, GEMM_THREADS, GEMM_SMEM, stream>>>(ma, mb, mc, md, p);
  count_launch();
  return launch_status();
}

// MoE experts, backward of the down projection + SwiGLU: for the rows of each group g
//   d(gate_up)[rows_g] = swiglu'(gate_up[rows_g]) applied to dy[rows_g] * W_down[g]      (W_down: [groups, D, I])
// d(act) never reaches memory (the dense MLP's SwiGLU-backward epilogue with the expert picked per tile). I % 8 == 0.
TLM_API int tlm_gemm_swiglu_bwd_grouped(const void* dy, const void* w_down, const void* gate_up, void* d_gate_up,
                                        const int* row_start, int groups, int R, int I, int D, long long lda,
                                        long long w_group_stride, int max_rows_per_group, cudaStream_t stream) {
  if (R <= 0 || I <= 0 || D <= 0 || groups <= 0) return 0;
  if (I % 8 != 0) return -4;
  Operand oa{dy, R, D, lda, false, 0, 0}, ob{w_down, I, D, I, true, groups, w_group_stride};
  CUtensorMap ma, mb, mc;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  e = build_map(&mb, ob, BN);
  if (e) return e;
  e = store_map_bf16(&mc, d_gate_up, R, 2LL * I, 2LL * I);
  if (e) return e;
  GemmParams p{};
  p.M = R; p.N = I; p.K = D; p.C = d_gate_up; p.ldc = 2LL * I; p.status = status_word(); p.split_k = 1; p.k_chunk = D;
  p.aux = (const __nv_bfloat16*)gate_up;
  p.groups = groups; p.row_start = row_start; p.group_mode = 1;
  if (use_pair_grouped(R, groups)) {
    p.max_tiles_m = (max_rows_per_group + 2 * BM - 1) / (2 * BM);
    static bool pconfigured = false;
    if (!pconfigured) {
      cudaError_t ce = cudaFuncSetAttribute(gemm_swiglu_bwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_PAIR);
      if (ce != cudaSuccess) return (int)ce;
      pconfigured = true;
    }
    const int pgrid = pair_grid((long long)groups * p.max_tiles_m * ((I + BN - 1) / BN));
    gemm_swiglu_bwd_pair_kernel<<<pgrid, GEMM_THREADS_WIDE, GEMM_SMEM_PAIR, stream>>>(ma, mb, mc, p);
    count_launch();
    return launch_status();
  }
  p.max_tiles_m = (max_rows_per_group + BM - 1) / BM;
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(gemm_swiglu_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  const int tiles = groups * p.max_tiles_m * ((I + BN - 1) / BN);
  const int grid = tiles < num_sms() ? tiles : num_sms();
  gemm_swiglu_bwd_kernel<<<grid, GEMM_THREADS_WIDE, GEMM_SMEM, stream>>>(ma, mb, mc, p);
  count_launch();
  return launch_status();
}

// Log-sum-exp statistics of logits = x [M, K] * w [N, K]^T without storing the logits (see GemmParams, EPI_LSE):
//   part [M, tiles] float2 (max, sum of exp(logit - max)) per 256-column tile, tiles = ceil(N / 256);
//   tgt_logit [M]: logit of column targets[row] (rows whose target is outside [0, N) keep their old value).
TLM_API int tlm_gemm_lse(const void* x, const void* w, int M, int N, int K, long long lda, long long ldb, void* part,
                         const long long* targets, float* tgt_logit, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (part == nullptr || targets == nullptr || tgt_logit == nullptr) return -6;
  Operand oa{x, M, K, lda, false, 0, 0}, ob{w, N, K, ldb, false, 1, (long long)N * K};
  CUtensorMap ma, mb;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  const bool pair = use_pair(M);
  e = build_map(&mb, ob, pair ? BN / 2 : BN);
  if (e) return e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = nullptr; p.ldc = 0; p.status = status_word(); p.groups = 0;
  p.split_k = 1; p.k_chunk = K;
  p.lse_part = (float2*)part; p.lse_tiles = (N + BN - 1) / BN; p.targets = targets; p.tgt_logit = tgt_logit;
  const int tiles = ((M + (pair ? 2 : 1) * BM - 1) / ((pair ? 2 : 1) * BM)) * ((N + BN - 1) / BN);
  return dispatch(false, false, EPI_LSE, ma, mb, p, tiles, stream, pair);
}

// dlogits [M, N] (bf16, row pitch ldc) = scale * (softmax(x w^T) - onehot(targets)) from the rows' log-sum-exp
// (see GemmParams, dl_*): the logits are recomputed tile by tile and leave as their own gradient.
// Requirements: ldc % 8 == 0 and a 16-byte aligned output (the tile stores go through TMA).
TLM_API int tlm_gemm_dlogits(const void* x, const void* w, void* dlogits, int M, int N, int K, long long lda, long long ldb,
                             long long ldc, const float* lse, const long long* targets, const float* scale,
                             long long ignore_index, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (lse == nullptr || targets == nullptr || scale == nullptr || ldc % 8 != 0 || (reinterpret_cast<uintptr_t>(dlogits) & 15)) return -6;
  Operand oa{x, M, K, lda, false, 0, 0}, ob{w, N, K, ldb, false, 1, (long long)N * K};
  CUtensorMap ma, mb;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  const bool pair = use_pair(M);
  e = build_map(&mb, ob, pair ? BN / 2 : BN);
  if (e) return e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = dlogits; p.ldc = ldc; p.status = status_word(); p.groups = 0;
  p.split_k = 1; p.k_chunk = K;
  p.dl_lse = lse; p.targets = targets; p.dl_scale = scale; p.dl_ignore = ignore_index;
  const int tiles = ((M + (pair ? 2 : 1) * BM - 1) / ((pair ? 2 : 1) * BM)) * ((N + BN - 1) / BN);
  return dispatch(false, false, EPI_BF16, ma, mb, p, tiles, stream, pair);
}

// C[M,N] = A * B^T with arbitrary operand majors.
//   a_mn = 0: A is [M,K] (lda); a_mn = 1: A is [K,M] (lda)
//   b_mn = 0: B is [N,K] (ldb); b_mn = 1: B is [K,N] (ldb)
//   epi: 0 bf16 store, 1 fp32 accumulate (C += ...), 2 fp32 store
TLM_API int tlm_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                     long long ldc, int a_mn, int b_mn, int epi, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.status = status_word(); p.groups = 0;
  if (!a_mn && !b_mn && epi == EPI_BF16) take_pending_waits(p);     // x W^T: may be the first reader of its weights
  const bool pair = use_pair(M) && p.wait_flags[0] == nullptr;
  Operand oa{A, M, K, lda, a_mn != 0, 0, 0}, ob{B, N, K, ldb, b_mn != 0, 1, (long long)N * K};
  CUtensorMap ma, mb;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  e = build_map(&mb, ob, pair ? BN / 2 : BN);
  if (e) return e;
  const int tile_m = pair ? 2 * BM : BM;
  int tiles = ((M + tile_m - 1) / tile_m) * ((N + BN - 1) / BN);
  p.split_k = 1; p.k_chunk = K;
  if (epi == EPI_F32_ACC && !g_deterministic) {
    // Weight gradients: few output tiles, long reduction. The persistent grid runs work items (tile x k-split)
    // of equal size in waves of one item per SM, so time ~ waves * (k-blocks per item + E), E = cost of one
    // epilogue pass (fp32 read-modify-write or red.global of a 128 KB tile) in k-block units (measured ~8).
    // Items keep at least 64 k-blocks.
    const int sms = pair ? num_sms() / 2 : num_sms();     // tile walkers
    const int kblocks = (K + BK - 1) / BK;
    static int min_kb = -1, e_cost = -1, cap = -1;
    if (min_kb < 0) {
      const char* v;
      min_kb = (v = getenv("TLM_SPLITK_MINKB")) ? atoi(v) : 64;
      e_cost = (v = getenv("TLM_SPLITK_E")) ? atoi(v) : 8;
      cap = (v = getenv("TLM_SPLITK_MAX")) ? atoi(v) : 16;
    }
    int max_split = kblocks / min_kb;
    if (max_split > cap) max_split = cap;
    int best = 1;
    double best_cost = 1e30;
    for (int sp = 1; sp <= (max_split > 1 ? max_split : 1); ++sp) {
      const long long items = (long long)tiles * sp;
      const long long waves = (items + sms - 1) / sms;
      const double cost = (double)waves * ((double)((kblocks + sp - 1) / sp) + (double)e_cost);
      if (cost < best_cost - 1e-9) { best_cost = cost; best = sp; }
    }
    if (best > 1) {
      const int per = (kblocks + best - 1) / best;
      p.k_chunk = per * BK;
      p.split_k = (kblocks + per - 1) / per;
    }
  }
  return dispatch(a_mn != 0, b_mn != 0, epi, ma, mb, p, tiles * p.split_k, stream, pair);
}

// Grouped forward / dgrad: rows of A and C are grouped (`row_start`, device,
// groups+1 ints, ascending, row_start[groups] == M); group g multiplies by
// B[g] ([N,K] K-major or [K,N] MN-major, `b_group_stride` elements apart).
// `max_rows_per_group` bounds the per-group tile count (a host-known bound,
// e.g. M); tiles beyond a group's real row count exit immediately.
TLM_API int tlm_gemm_grouped_rows(const void* A, const void* B, void* C, const int* row_start, int groups, int M,
                                  int N, int K, long long lda, long long ldb, long long b_group_stride,
                                  long long ldc, int b_mn, int epi, int max_rows_per_group, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || groups <= 0) return 0;
  Operand oa{A, M, K, lda, false, 0, 0}, ob{B, N, K, ldb, b_mn != 0, groups, b_group_stride};
  CUtensorMap ma, mb;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  const bool pair = use_pair_grouped(M, groups);
  e = build_map(&mb, ob, pair ? BN / 2 : BN);
  if (e) return e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.status = status_word();
  p.groups = groups; p.row_start = row_start; p.group_mode = 1;
  p.max_tiles_m = (max_rows_per_group + (pair ? 2 : 1) * BM - 1) / ((pair ? 2 : 1) * BM);
  int tiles = groups * p.max_tiles_m * ((N + BN - 1) / BN);
  return dispatch(false, b_mn != 0, epi, ma, mb, p, tiles, stream, pair);
}

// Paired grouped GEMMs for the MoE gate / up projections. `W` holds 2 * groups matrices [I, D] (gate of
// group g at g, up at groups + g), `w_group_stride` elements apart.
//   dgrad == 0:  C[R, 2 I] (ldc) = A[R, D] * [W_g ; W_{groups+g}]^T      gate | up side by side, I % 256 == 0
//   dgrad == 1:  C[R, D]  (ldc) = A[R, 2 I] * [W_g ; W_{groups+g}]       both data gradients summed, I % 64 == 0
TLM_API int tlm_gemm_grouped_pair(const void* A, const void* W, void* C, const int* row_start, int groups, int R, int I,
                                  int D, long long lda, long long w_group_stride, long long ldc, int dgrad,
                                  int max_rows_per_group, cudaStream_t stream) {
  if (R <= 0 || I <= 0 || D <= 0 || groups <= 0) return 0;
  if ((!dgrad && I % BN != 0) || (dgrad && I % BK != 0)) return -4;
  const int N = dgrad ? D : 2 * I, K = dgrad ? 2 * I : D;
  Operand oa{A, R, K, lda, false, 0, 0};
  // forward: B K-major [I rows, D]; dgrad: B MN-major, stored [I (reduction), D (output)]
  Operand ob{W, dgrad ? D : I, dgrad ? I : D, D, dgrad != 0, 2LL * groups, w_group_stride};
  CUtensorMap ma, mb;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  const bool pair = use_pair_grouped(R, groups);
  e = build_map(&mb, ob, pair ? BN / 2 : BN);
  if (e) return e;
  GemmParams p{};
  p.M = R; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.status = status_word();
  p.groups = groups; p.row_start = row_start; p.group_mode = 1;
  p.max_tiles_m = (max_rows_per_group + (pair ? 2 : 1) * BM - 1) / ((pair ? 2 : 1) * BM);
  if (dgrad) p.pair_k = I; else p.pair_n = I;
  int tiles = groups * p.max_tiles_m * ((N + BN - 1) / BN);
  return dispatch(false, dgrad != 0, EPI_BF16, ma, mb, p, tiles, stream, pair);
}

// Same as tlm_gemm_grouped_rows with a bf16 store, but output row r goes to dst_ptrs[dest_rank[r]] row dest_row[r]
// (row pitch ldc; rows with dest_rank < 0 are dropped): the expert-parallel combine done by the GEMM epilogue.
TLM_API int tlm_gemm_grouped_rows_scatter(const void* A, const void* B, const int* row_start, int groups, int M, int N,
                                          int K, long long lda, long long ldb, long long b_group_stride, long long ldc,
                                          int b_mn, int max_rows_per_group, const int* dest_rank,
                                          const long long* dest_row, void* const* dst_ptrs, int n_dst,
                                          long long dst_rows, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || groups <= 0) return 0;
  if (n_dst < 1 || n_dst > MAX_HEAD_DST || dest_rank == nullptr || dest_row == nullptr || ldc % 8 != 0) return -6;
  Operand oa{A, M, K, lda, false, 0, 0}, ob{B, N, K, ldb, b_mn != 0, groups, b_group_stride};
  CUtensorMap ma, mb;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  const bool pair = use_pair_grouped(M, groups);
  e = build_map(&mb, ob, pair ? BN / 2 : BN);
  if (e) return e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = nullptr; p.ldc = ldc; p.status = status_word();
  p.groups = groups; p.row_start = row_start; p.group_mode = 1;
  p.max_tiles_m = (max_rows_per_group + (pair ? 2 : 1) * BM - 1) / ((pair ? 2 : 1) * BM);
  p.rs_rank = dest_rank; p.rs_row = dest_row; p.rs_rows = dst_rows;
  for (int i = 0; i < n_dst; ++i) p.rs_dst[i] = dst_ptrs[i];
  int tiles = groups * p.max_tiles_m * ((N + BN - 1) / BN);
  return dispatch(false, b_mn != 0, EPI_ROWS, ma, mb, p, tiles, stream, pair);
}

// Grouped wgrad: C[g] ([M,N] fp32, `c_group_stride` apart) += A[rows_g, M]^T * B[rows_g, N]
// where rows_g = [row_start[g], row_start[g+1]) is the reduction range.
// A is stored [R, M] and B [R, N] (both MN-major with respect to the product).
TLM_API int tlm_gemm_grouped_k(const void* A, const void* B, void* C, const int* row_start, int groups, int R,
                               int M, int N, long long lda, long long ldb, long long ldc, long long c_group_stride,
                               int epi, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || R <= 0 || groups <= 0) return 0;
  Operand oa{A, M, R, lda, true, 0, 0}, ob{B, N, R, ldb, true, 1, (long long)R * N};
  CUtensorMap ma, mb;
  int e = build_map(&ma, oa, BM);
  if (e) return e;
  e = build_map(&mb, ob, BN);
  if (e) return e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = R; p.C = C; p.ldc = ldc; p.status = status_word();
  p.groups = groups; p.row_start = row_start; p.group_mode = 2; p.c_group_stride = c_group_stride;
  int tiles = groups * ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  return dispatch(true, true, epi, ma, mb, p, tiles, stream);
}
