"""Exchange buffers of the peer-memory paths are cached per (key, shape) and never replaced: a recorded CUDA
graph keeps writing to the buffers of the shape it was recorded with (their local and peer addresses are in
its kernel arguments and tensor maps), so a batch of another shape must get buffers of its own."""
import torch


class _FakeExchange:
    made = 0

    def __init__(self, shape, group, device):
        type(self).made += 1
        self.tensor = torch.zeros(shape)
        self.serial = type(self).made


def test_ulysses_receive_buffers_are_keyed_by_shape_and_kept(monkeypatch):
    from train_large_model_from_scratch_b200.parallel.sequence_parallel import ulysses_peer
    monkeypatch.setattr(ulysses_peer, "_Exchange", _FakeExchange)
    st = object.__new__(ulysses_peer.PeerState)
    st.group, st.buffers = None, {}
    full = st.buffer(("layer0", "qkv"), (8, 4096, 4, 64), "cpu")
    ragged = st.buffer(("layer0", "qkv"), (3, 4096, 4, 64), "cpu")       # last batch of an epoch / evaluation batch
    again = st.buffer(("layer0", "qkv"), (8, 4096, 4, 64), "cpu")
    assert again is full and ragged is not full                          # the recorded shape keeps ITS buffer
    assert tuple(full.tensor.shape) == (8, 4096, 4, 64) and tuple(ragged.tensor.shape) == (3, 4096, 4, 64)
    assert len(st.buffers) == 2


def test_moe_receive_buffers_are_keyed_by_shape_and_kept(monkeypatch):
    from train_large_model_from_scratch_b200.parallel import symm
    from train_large_model_from_scratch_b200.parallel.expert_parallel import peer
    monkeypatch.setattr(symm, "symm_alloc", lambda n, dt, dev: torch.zeros(n, dtype=dt))
    monkeypatch.setattr(symm, "_Peer", lambda t, g: ("peer", t.data_ptr()))
    pm = object.__new__(peer.PeerMoE)
    pm.group, pm.dev, pm.buffers = None, "cpu", {}
    a = pm.buffer(("l0", "disp"), 64, 16)
    b = pm.buffer(("l0", "disp"), 24, 16)
    c = pm.buffer(("l0", "disp"), 64, 16)
    assert c is a and b is not a and a[0].shape == (64, 16) and b[0].shape == (24, 16)
    assert a[1][1] == a[0].data_ptr()                                    # the peer handle belongs to this storage


def test_fused_ulysses_path_conditions_include_replicated_kv_heads(monkeypatch):
    """Which head / rank combinations ride on the GEMM and attention epilogues (`ulysses_peer.fused_ok`): whole KV heads
    per rank, or whole ranks per KV head (replication), head dims 64 / 128 and 32-row multiples only."""
    from train_large_model_from_scratch_b200.parallel.sequence_parallel import ulysses_peer
    monkeypatch.delenv("TLM_SP_FUSED", raising=False)
    assert ulysses_peer.fused_ok(16, 8, 8, 64, 4096)          # one KV head per rank
    assert ulysses_peer.fused_ok(16, 8, 2, 128, 64)           # four KV heads per rank
    assert ulysses_peer.fused_ok(32, 4, 8, 64, 512)           # each KV head replicated to two ranks
    assert ulysses_peer.fused_ok(4, 1, 2, 64, 128)
    assert not ulysses_peer.fused_ok(32, 4, 8, 32, 512)       # head dim 32: stand-alone scatter kernels / library path
    assert not ulysses_peer.fused_ok(12, 4, 8, 64, 512)       # query heads do not divide
    assert not ulysses_peer.fused_ok(24, 3, 2, 64, 512)       # neither whole heads per rank nor whole ranks per head
    assert not ulysses_peer.fused_ok(16, 8, 8, 64, 100)       # rows per rank not a multiple of 32
    monkeypatch.setenv("TLM_SP_FUSED", "0")
    assert not ulysses_peer.fused_ok(16, 8, 8, 64, 4096)


def test_replicated_kv_gradient_slots_sum_to_the_packed_layout():
    """The sequence owner's packed gradient buffer under KV replication has one dK and one dV slot per source rank
    (`n_q + 2 sp` heads); summing each head's adjacent replicas must give `[dQ | dK | dV]` with `n_kv` heads each.
    Same arithmetic as `_UlyssesAttention.backward`."""
    import torch
    B, T_l, n_q, n_kv, sp, hd = 2, 3, 8, 2, 4, 4
    rep = sp // n_kv
    g = torch.Generator().manual_seed(0)
    dq = torch.randn(B, T_l, n_q, hd, generator=g)
    parts_k = torch.randn(B, T_l, sp, hd, generator=g)         # slot r: rank r's partial dK of KV head r // rep
    parts_v = torch.randn(B, T_l, sp, hd, generator=g)
    d = torch.cat([dq, parts_k, parts_v], dim=2)
    dkv = d[:, :, n_q:].reshape(B, T_l, 2 * n_kv, rep, hd).float().sum(3)
    packed = torch.cat([d[:, :, :n_q], dkv], dim=2)
    for j in range(n_kv):
        torch.testing.assert_close(packed[:, :, n_q + j], parts_k[:, :, j * rep:(j + 1) * rep].sum(2))
        torch.testing.assert_close(packed[:, :, n_q + n_kv + j], parts_v[:, :, j * rep:(j + 1) * rep].sum(2))
    assert packed.shape == (B, T_l, n_q + 2 * n_kv, hd)
