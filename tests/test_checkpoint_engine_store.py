"""Host-memory checkpoint engine: bucketing, several receivers, consecutive rounds, key clean-up."""
import threading

import torch

from twinkle_b200.checkpoint_engine import StoreCheckpointEngine, make_engine


def test_store_engine_two_receivers_two_rounds():
    send = StoreCheckpointEngine('send', n_receivers=2, bucket_bytes=1500)
    recv = [make_engine('store', 'recv', store_port=send.port, n_receivers=2, receiver_index=i) for i in range(2)]
    rounds = [{f'layer.{i}.weight': torch.randn(16, 9) for i in range(7)} | {'ids': torch.arange(11), 'empty': torch.empty(0, 4)},
              {'lora_A': torch.randn(8, 32), 'lora_B': torch.zeros(32, 8)}]
    for weights in rounds:
        got = [dict(), dict()]

        def take(i):
            for k, v in recv[i].receive_weights():
                got[i][k] = v.clone()

        threads = [threading.Thread(target=take, args=(i, )) for i in range(2)]
        for t in threads:
            t.start()
        stats = send.send_weights(weights.items())
        for t in threads:
            t.join(timeout=30)
        assert stats['bytes'] > 0
        for g in got:
            assert list(g) == list(weights)                                   # order kept
            for k, v in weights.items():
                want = v.to(torch.bfloat16) if v.dtype == torch.float32 else v     # fp32 travels as bf16
                assert g[k].dtype == want.dtype and g[k].shape == want.shape and torch.equal(g[k], want)
    assert send.store.num_keys() <= 1 + 2 * 2 * 8, 'bucket payloads must be deleted once acknowledged'
    assert not any(send.store.check([f'r{r}/bucket/{b}']) for r in range(2) for b in range(8))


def test_mixin_requires_prepare():
    import pytest
    from twinkle_b200.checkpoint_engine import CheckpointEngineMixin

    class S(CheckpointEngineMixin):
        def update_weights(self, weights, peft_config=None):
            self.seen = dict(weights)

    s = S()
    with pytest.raises(RuntimeError, match='prepare_checkpoint_engine'):
        s._receive_weights()
