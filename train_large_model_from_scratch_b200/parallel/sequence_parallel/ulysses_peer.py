"""Ulysses seq<->head exchanges as direct stores into peer memory (CUDA).

Replaces, on the GPU, the pack -> `all_to_all_single` -> unpack sequence of
`ulysses.py` (and the reference's `model/modules/attn.py:143-171`). On the fused
path (`_UlyssesAttention`) all four exchanges of a layer happen inside compute
kernels: QKV projection + RoPE + seq->head in the GEMM epilogue; head->seq of O
in the attention epilogue; in backward seq->head of dO in the epilogue of the
output projection's data-gradient GEMM, and head->seq of the packed gradient
(with the transposed rotation) from the attention-backward kernels themselves.
Shapes the head-scatter GEMM epilogue does not take (head dim 32, sequence
chunks that are not a multiple of 32) use `_SeqToHead` / `_HeadToSeq`, whose
exchanges are one scatter kernel each (`csrc/ulysses.cu`). Every exchange ends
with a flag barrier:

  forward   qkv  [B, T_l, Hq+2Hkv, hd] --RoPE + scatter--> every head owner's
            [B, T_full, q_l+2kv_l, hd]; attention; o [B, T_full, q_l, hd]
            --scatter--> every sequence owner's [B, T_l, Hq, hd]
  backward  the transposed routes; the transposed RoPE rides on the way back.

RoPE is applied inside the first scatter, so the separate RoPE pass and its
read + write of the qkv tensor disappear as well.

Receive buffers live in symmetric memory, one set per attention layer, created
at the layer's first call (a collective rendezvous, same order on every rank)
and reused by later steps. They double as the tensors saved for backward. Reuse
is safe without extra handshakes: a peer can only reach the next write into a
buffer after an exchange that this rank completes after its last read of it.

Only head plans without KV replication (`Hkv % sp == 0`) take this path; the
others use the NCCL path, where replicated KV gradients are summed by autograd.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ...ops import native
from . import ulysses


def _fresh(t: torch.Tensor) -> torch.Tensor:
    """A new tensor object over the same storage. The receive buffers live for the whole run; handing the
    cached object itself to autograd as a Function's output would tie it to one step's graph (history set on
    it in one step is still there in the next, with that step's stream)."""
    return t.view(t.shape)


class _Exchange:
    """One symmetric receive buffer + its peers' addresses."""

    def __init__(self, shape, group, device):
        from ..symm import symm_alloc, _Peer
        n = 1
        for s in shape:
            n *= s
        self.tensor = symm_alloc(n, torch.bfloat16, device).view(shape)
        self.peer = _Peer(self.tensor, group)


class PeerState:
    """Per-process state of the peer path for one SEP group."""

    _instance = None

    def __init__(self, group):
        from ..symm import alloc_flags, _Peer
        self.group = group
        self.sp = dist.get_world_size(group)
        self.me = dist.get_rank(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.flags_t = alloc_flags(dev)
        self.flags = _Peer(self.flags_t, group)
        self.buffers: dict = {}
        self.tables: dict = {}
        dist.barrier(group=group)

    @classmethod
    def get(cls, group) -> "PeerState":
        if cls._instance is None or cls._instance.group is not group:
            cls._instance = cls(group)
        return cls._instance

    def buffer(self, key, shape, device) -> _Exchange:
        """The receive buffer of `key` for this shape. Buffers are cached per (key, shape) and never freed: a
        recorded CUDA graph has the local and peer addresses of the buffers of ITS shape in its kernel arguments
        and tensor maps, so a call with another shape (a ragged last batch, an evaluation batch) must get a
        buffer of its own instead of replacing the one the recording still writes to."""
        key = (key, tuple(int(s) for s in shape))
        ex = self.buffers.get(key)
        if ex is None:
            ex = _Exchange(shape, self.group, device)
            self.buffers[key] = ex
        return ex

    def table(self, key, rows, device) -> torch.Tensor:
        t = self.tables.get(key)
        if t is None:
            t = torch.tensor(rows, dtype=torch.int32, device=device).contiguous()
            self.tables[key] = t
        return t

    def barrier(self) -> None:
        f = self.flags
        native._check(native.lib().tlm_peer_barrier(f.ptr_array, f.rank, f.n, 0, native._stream()), "peer_barrier")


def supported(n_q: int, n_kv: int, sp: int, hd: int) -> bool:
    return n_q % sp == 0 and n_kv % sp == 0 and hd % 16 == 0


def _scatter(st: PeerState, src: torch.Tensor, ex: _Exchange, table: torch.Tensor, mode: int, cos, sin, pos0: int):
    B, Ts, Hs, hd = src.shape
    Hd = ex.tensor.shape[2]
    native._check(native.lib().tlm_peer_scatter_heads(
        src.data_ptr(), ex.peer.ptr_array, table.data_ptr(), native._ptr(cos), native._ptr(sin), mode, B, Ts, Hs, Hd, hd,
        st.sp, st.me, table.shape[0], pos0, native._stream()), "peer_scatter_heads")
    st.barrier()


class _SeqToHead(torch.autograd.Function):
    """qkv (un-rotated) `[B, T_l, Hq+2Hkv, hd]` -> rotated `[B, T_full, q_l+2kv_l, hd]` of my heads."""

    @staticmethod
    def forward(ctx, qkv, n_q, n_kv, cos_l, sin_l, cos_f, sin_f, layer_key, group):
        st = PeerState.get(group)
        sp, me = st.sp, st.me
        B, T_l, Ht, hd = qkv.shape
        plans, q_l, kv_l = ulysses.head_plan(n_q, n_kv, sp)
        hpr = q_l + 2 * kv_l
        rows = []
        for dest, plan in enumerate(plans):
            for slot, h in enumerate(plan):
                rows.append([h, dest, slot, 1 if h < n_q + n_kv else 0])
        table = st.table(("s2h", n_q, n_kv), rows, qkv.device)
        ex = st.buffer((layer_key, "qkv"), (B, sp * T_l, hpr, hd), qkv.device)
        _scatter(st, qkv.contiguous(), ex, table, 0, cos_l, sin_l, 0)
        ctx.meta = (n_q, n_kv, q_l, kv_l, layer_key, group, B, T_l, hd)
        ctx.save_for_backward(cos_f, sin_f)
        return _fresh(ex.tensor)

    @staticmethod
    def backward(ctx, d_full):
        n_q, n_kv, q_l, kv_l, layer_key, group, B, T_l, hd = ctx.meta
        cos_f, sin_f = ctx.saved_tensors
        st = PeerState.get(group)
        table = _dqkv_table(st, n_q, n_kv, q_l, kv_l, d_full.device)
        ex = st.buffer((layer_key, "dqkv"), (B, T_l, n_q + 2 * n_kv, hd), d_full.device)
        _scatter(st, d_full.contiguous(), ex, table, 1, cos_f, sin_f, 0)
        return _fresh(ex.tensor), None, None, None, None, None, None, None, None


class _HeadToSeq(torch.autograd.Function):
    """attention output `[B, T_full, q_l, hd]` (my heads) -> `[B, T_l, Hq, hd]` (my rows)."""

    @staticmethod
    def forward(ctx, o, n_q, layer_key, group):
        st = PeerState.get(group)
        sp, me = st.sp, st.me
        B, T_full, q_l, hd = o.shape
        rows = [[i, 0, me * q_l + i, 0] for i in range(q_l)]
        table = st.table(("h2s_o", n_q), rows, o.device)
        ex = st.buffer((layer_key, "o"), (B, T_full // sp, n_q, hd), o.device)
        _scatter(st, o.contiguous(), ex, table, 1, None, None, 0)
        ctx.meta = (n_q, q_l, layer_key, group, B, T_full, hd)
        return _fresh(ex.tensor)

    @staticmethod
    def backward(ctx, d_seq):
        n_q, q_l, layer_key, group, B, T_full, hd = ctx.meta
        st = PeerState.get(group)
        sp = st.sp
        rows = []
        for dest in range(sp):
            for i in range(q_l):
                rows.append([dest * q_l + i, dest, i, 0])
        table = st.table(("s2h_do", n_q), rows, d_seq.device)
        ex = st.buffer((layer_key, "do"), (B, T_full, q_l, hd), d_seq.device)
        _scatter(st, d_seq.contiguous(), ex, table, 0, None, None, 0)
        return _fresh(ex.tensor), None, None, None


def _dqkv_table(st: PeerState, n_q, n_kv, q_l, kv_l, device) -> torch.Tensor:
    """head->seq route of the packed gradient: my local slot -> packed head index on the
    sequence owner; q and k slots get the transposed rotation."""
    me = st.me
    rows = [[i, 0, me * q_l + i, 2] for i in range(q_l)]
    rows += [[q_l + i, 0, n_q + me * kv_l + i, 2] for i in range(kv_l)]
    rows += [[q_l + kv_l + i, 0, n_q + n_kv + me * kv_l + i, 0] for i in range(kv_l)]
    return st.table(("h2s_dqkv", n_q, n_kv), rows, device)


class _UlyssesAttention(torch.autograd.Function):
    """The whole attention block under Ulysses as one autograd node, `h [B*T_l, D]` -> `[B*T_l, D]`, with all
    four exchanges of a layer inside compute kernels:

      forward   QKV GEMM epilogue: RoPE + packed layout + seq->head stores into the head owners' memory;
                attention epilogue: head->seq stores of O into the sequence owners' memory; output GEMM.
      backward  output-projection dgrad GEMM epilogue: seq->head stores of dO into the head owners' memory;
                attention backward: dQ (while it is converted from its fp32 accumulator) and dK / dV (as they
                leave tensor memory) get the transposed RoPE and are stored head->seq into the sequence owners'
                packed gradient buffer, which feeds the QKV weight- and data-gradient GEMMs.

    No stand-alone scatter kernel is left; each exchange ends with a flag barrier.

    Fewer KV heads than ranks (`n_kv < sp`, `sp % n_kv == 0`): KV head j is replicated to the `sp / n_kv` ranks that
    own its query heads (the QKV epilogue stores its tile once per owner), every rank attends with one local KV
    head, and the partial dK / dV of the replicas come back into separate slots of the packed gradient buffer
    (`n_q + 2 sp` heads), where the sequence owner sums them before the QKV gradient GEMMs."""

    @staticmethod
    def forward(ctx, h, w_qkv, w_out, n_q, n_kv, hd, B, T_l, cs_l, cos_f, sin_f, layer_key, group):
        from ...ops import attention_cuda
        st = PeerState.get(group)
        sp, me = st.sp, st.me
        kv_rep = sp // n_kv if n_kv < sp else 1
        q_l, kv_l = n_q // sp, (1 if kv_rep > 1 else n_kv // sp)
        hpr = q_l + 2 * kv_l
        T_full = sp * T_l
        ex_qkv = st.buffer((layer_key, "qkv"), (B, T_full, hpr, hd), h.device)
        native.gemm_heads(h, w_qkv, False, ex_qkv.peer.ptr_array, sp, B, T_l, T_full, hpr, me * T_l, n_q, n_kv,
                          q_l, kv_l, hd, n_q + n_kv, cs_l, kv_rep)
        st.barrier()
        qkv_l = ex_qkv.tensor
        ex_o = st.buffer((layer_key, "o"), (B, T_l, n_q, hd), h.device)
        o, lse = attention_cuda.fwd_scatter(qkv_l, q_l, kv_l, ex_o.peer.ptr_array, sp, T_l, n_q, me * q_l)
        st.barrier()
        o_seq = ex_o.tensor.view(B * T_l, n_q * hd)
        ctx.meta = (n_q, n_kv, q_l, kv_l, hd, layer_key, group, B, T_l)
        ctx.w_qkv, ctx.w_out = w_qkv, w_out
        ctx.save_for_backward(h, qkv_l, o, lse, o_seq, cos_f, sin_f)
        return native.gemm_nt(o_seq, w_out)

    @staticmethod
    def backward(ctx, dy):
        from ...ops import attention_cuda
        from ...ops.functional import _main_grad
        n_q, n_kv, q_l, kv_l, hd, layer_key, group, B, T_l = ctx.meta
        h, qkv_l, o, lse, o_seq, cos_f, sin_f = ctx.saved_tensors
        w_qkv, w_out = ctx.w_qkv, ctx.w_out
        st = PeerState.get(group)
        sp, me = st.sp, st.me
        T_full = sp * T_l
        dy = dy.contiguous()
        native.gemm_tn_accum(dy, o_seq, _main_grad(w_out))
        ex_do = st.buffer((layer_key, "do"), (B, T_full, q_l, hd), dy.device)
        native.gemm_heads(dy, w_out, True, ex_do.peer.ptr_array, sp, B, T_l, T_full, q_l, me * T_l, n_q, 0, q_l, 1,
                          hd, 0, None)
        st.barrier()
        kv_rep = sp // n_kv if n_kv < sp else 1
        n_kv_slots = sp if kv_rep > 1 else n_kv           # replicated KV heads: one dK and one dV slot per source rank
        Ht = n_q + 2 * n_kv_slots
        ex_d = st.buffer((layer_key, "dqkv"), (B, T_l, Ht, hd), dy.device)
        attention_cuda.bwd_scatter(ex_do.tensor, qkv_l, o, lse, q_l, kv_l, (cos_f, sin_f), ex_d.peer.ptr_array, sp, T_l, Ht,
                                   me * q_l, n_q + me * kv_l, n_q + n_kv_slots + me * kv_l)
        st.barrier()
        if kv_rep > 1:
            # rank j * kv_rep + c holds replica c of KV head j: slots of one head are adjacent, sum them in fp32
            d = ex_d.tensor
            dkv = d[:, :, n_q:].reshape(B, T_l, 2 * n_kv, kv_rep, hd).float().sum(3).to(d.dtype)
            d2 = torch.cat([d[:, :, :n_q], dkv], dim=2).view(B * T_l, -1)
        else:
            d2 = ex_d.tensor.view(B * T_l, -1)
        native.gemm_tn_accum(d2, h, _main_grad(w_qkv))
        dh = native.gemm_nn(d2, w_qkv) if ctx.needs_input_grad[0] else None
        return (dh,) + (None,) * 12


def attention_block(h, w_qkv, w_out, n_q, n_kv, hd, B, T_l, cs_l, cos_f, sin_f, layer_key, group):
    """`cs_l` = `native.rope_table_fp16` of this rank's positions; `cos_f` / `sin_f`: fp32 tables of the full sequence."""
    return _UlyssesAttention.apply(h, w_qkv, w_out, n_q, n_kv, hd, B, T_l, cs_l, cos_f.contiguous(), sin_f.contiguous(),
                                   layer_key, group)


def fused_ok(n_q: int, n_kv: int, sp: int, hd: int, T_l: int) -> bool:
    """Shapes for which the exchanges ride on the GEMM epilogues."""
    import os
    heads_ok = n_q % sp == 0 and (n_kv % sp == 0 or (sp % n_kv == 0 and (n_q // n_kv) % (sp // n_kv) == 0))
    return (heads_ok and native.heads_epilogue_ok(hd, T_l, sp)
            and os.environ.get("TLM_SP_FUSED", "1") != "0")       # 0: keep the stand-alone scatter kernels


def seq_to_head(qkv, n_q, n_kv, cos_l, sin_l, cos_f, sin_f, layer_key, group):
    return _SeqToHead.apply(qkv, n_q, n_kv, cos_l, sin_l, cos_f, sin_f, layer_key, group)


def head_to_seq(o, n_q, layer_key, group):
    return _HeadToSeq.apply(o, n_q, layer_key, group)
