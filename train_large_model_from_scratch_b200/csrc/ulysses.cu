// Ulysses sequence parallelism over NVLink peer memory: the seq<->head
// re-layout is done by ONE kernel per exchange that reads the local tensor once
// and stores every 16-byte piece directly into the owning rank's buffer
// (symmetric memory), applying RoPE (or its transpose, in backward) on the way.
// There is no pack / all-to-all / unpack sequence and no intermediate copy.
//
//   mode 0, seq -> head   (qkv in forward, dO in backward)
//       src [B, Ts, Hs, hd] : my sequence chunk, all heads
//       entry e = (src_head, dest_rank, dst_head, rotate) -> dst[dest][b, me*Ts + t, dst_head, :]
//       dst  [B, sp*Ts, Hd, hd]
//   mode 1, head -> seq   (attention output in forward, dqkv in backward)
//       src [B, Ts, Hs, hd] : the whole sequence, my heads;  row t belongs to rank t / (Ts/sp)
//       entry e = (src_head, -, dst_head, rotate)            -> dst[t / Tl][b, t % Tl, dst_head, :]
//       dst  [B, Ts/sp, Hd, hd]
// rotate: 0 none, 1 RoPE, 2 transposed RoPE; the table row is `pos0 + t`.
// Completion is published afterwards with the flag barrier of collectives.cu.
#include "common.cuh"

namespace tlm {

struct ScatterPeers { void* p[16]; };

struct ScatterParams {
  const __nv_bfloat16* src;
  ScatterPeers dst;
  const int4* table;        // device, n_entries
  const float* cosT;        // [*, hd]
  const float* sinT;
  int mode, B, Ts, Hs, Hd, hd, sp, me, n_entries, pos0;
};

__global__ void peer_scatter_heads_kernel(const ScatterParams p) {
  const int half = p.hd / 2, vec = half / 8;
  const long long total = (long long)p.B * p.Ts * p.n_entries * vec;
  const int Tl = p.mode == 1 ? p.Ts / p.sp : p.Ts;
  const int Td = p.mode == 1 ? Tl : p.sp * p.Ts;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec);
    long long r = i / vec;
    const int e = (int)(r % p.n_entries); r /= p.n_entries;
    const int t = (int)(r % p.Ts);
    const int b = (int)(r / p.Ts);
    const int4 ent = p.table[e];
    const int j = v * 8;
    const __nv_bfloat16* s = p.src + (((long long)b * p.Ts + t) * p.Hs + ent.x) * p.hd + j;
    uint4 lo = *reinterpret_cast<const uint4*>(s), hi = *reinterpret_cast<const uint4*>(s + half);
    if (ent.w != 0) {
      const float* c = p.cosT + (long long)(p.pos0 + t) * p.hd + j;
      const float* sn = p.sinT + (long long)(p.pos0 + t) * p.hd + j;
      uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = unpack_bf16(lw[k]), bb = unpack_bf16(hw[k]);
        const float cl0 = c[2 * k], cl1 = c[2 * k + 1], ch0 = c[half + 2 * k], ch1 = c[half + 2 * k + 1];
        const float sl0 = sn[2 * k], sl1 = sn[2 * k + 1], sh0 = sn[half + 2 * k], sh1 = sn[half + 2 * k + 1];
        float y0, y1, z0, z1;
        if (ent.w == 1) {
          y0 = a.x * cl0 - bb.x * sl0; y1 = a.y * cl1 - bb.y * sl1;
          z0 = bb.x * ch0 + a.x * sh0; z1 = bb.y * ch1 + a.y * sh1;
        } else {
          y0 = a.x * cl0 + bb.x * sh0; y1 = a.y * cl1 + bb.y * sh1;
          z0 = bb.x * ch0 - a.x * sl0; z1 = bb.y * ch1 - a.y * sl1;
        }
        lw[k] = pack_bf16(y0, y1); hw[k] = pack_bf16(z0, z1);
      }
      lo = make_uint4(lw[0], lw[1], lw[2], lw[3]); hi = make_uint4(hw[0], hw[1], hw[2], hw[3]);
    }
    int dest, trow;
    if (p.mode == 1) { dest = t / Tl; trow = t - dest * Tl; } else { dest = ent.y; trow = p.me * p.Ts + t; }
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.dst.p[dest]) + (((long long)b * Td + trow) * p.Hd + ent.z) * p.hd + j;
    *reinterpret_cast<uint4*>(d) = lo;
    *reinterpret_cast<uint4*>(d + half) = hi;
  }
}

}  // namespace tlm

using namespace tlm;

TLM_API int tlm_peer_scatter_heads(const void* src, void* const* dst_ptrs, const void* table, const float* cosT,
                                   const float* sinT, int mode, int B, int Ts, int Hs, int Hd, int hd, int sp, int me,
                                   int n_entries, int pos0, cudaStream_t st) {
  if (sp > 16 || hd % 16 != 0) return -6;
  if (mode == 1 && Ts % sp != 0) return -7;
  ScatterParams p{};
  p.src = (const __nv_bfloat16*)src;
  for (int i = 0; i < sp; ++i) p.dst.p[i] = dst_ptrs[i];
  p.table = (const int4*)table; p.cosT = cosT; p.sinT = sinT;
  p.mode = mode; p.B = B; p.Ts = Ts; p.Hs = Hs; p.Hd = Hd; p.hd = hd; p.sp = sp; p.me = me; p.n_entries = n_entries; p.pos0 = pos0;
  long long items = (long long)B * Ts * n_entries * (hd / 16);
  long long blocks = (items + 255) / 256;
  if (blocks > 16LL * num_sms()) blocks = 16LL * num_sms();
  if (blocks < 1) return 0;
  peer_scatter_heads_kernel<<<(int)blocks, 256, 0, st>>>(p);
  count_launch();
  return launch_status();
}
