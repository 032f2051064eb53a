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
