"""Bounded device-side waits: a cross-GPU barrier whose peer never arrives gives up after its limit, records a
status word that the host reads, and leaves the context usable.  No rank is killed and nothing faults: the "peer"
is simply a flag that nobody writes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_barrier_wait_runs_out_and_reports():
    from twinkle_b200 import ops
    E = ops.ext()
    E.read_and_clear_error()
    mine, _, _ = E.symm_alloc(4096)        # flags this rank waits on
    peer, _, _ = E.symm_alloc(4096)        # stands in for the peer's flag buffer: this rank writes its arrival there
    mine.zero_()
    peer.zero_()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    E.symm_barrier([mine.data_ptr(), peer.data_ptr()], 0, 1, 200)   # rank 0 of 2, epoch 1, 200 ms limit
    b.record()
    torch.cuda.synchronize()
    waited = a.elapsed_time(b)
    assert 150 < waited < 2000, waited
    assert int(peer.view(torch.int32)[0]) == 1     # the arrival was published before the wait
    # while the error is pending, later barriers return at once instead of waiting again
    a.record()
    E.symm_barrier([mine.data_ptr(), peer.data_ptr()], 0, 2, 200)
    E.symm_barrier([mine.data_ptr(), peer.data_ptr()], 0, 3, 200)
    b.record()
    torch.cuda.synchronize()
    assert a.elapsed_time(b) < 100
    assert E.read_and_clear_error() == 5           # ERR_PEER_FLAG, reported once
    # the context is intact: kernels still run and give right answers
    x = torch.randn(256, 256, device='cuda').bfloat16()
    y = E.gemm(x, x, 'nt')
    assert torch.isfinite(y.float()).all()
    assert E.read_and_clear_error() == 0


def test_model_step_raises_on_pending_device_error():
    """The training API surfaces a pending status word as a Python exception at the next gradient-norm check."""
    from twinkle_b200 import ops
    from twinkle_b200.model import TransformersModel
    from twinkle_b200.models.config import preset
    E = ops.ext()
    cfg = preset('qwen3-8b', num_hidden_layers=1, hidden_size=256, intermediate_size=512, num_attention_heads=2, num_key_value_heads=1, vocab_size=512)
    m = TransformersModel(config=cfg, device='cuda', seed=0)
    m.set_optimizer('AdamW', lr=1e-3)
    feats = [{'input_ids': list(range(1, 65)), 'labels': list(range(2, 66))}]
    m.forward_backward(inputs=feats)
    mine, _, _ = E.symm_alloc(4096)
    peer, _, _ = E.symm_alloc(4096)
    mine.zero_()
    E.symm_barrier([mine.data_ptr(), peer.data_ptr()], 0, 1, 100)   # leaves ERR_PEER_FLAG behind
    with pytest.raises(RuntimeError, match='bounded wait'):
        m.clip_grad_and_step(max_grad_norm=1.0)
    m.forward_backward(inputs=feats)                                 # the next step is clean again
    m.clip_grad_and_step(max_grad_norm=1.0)
