"""T8 (CPU part): the async trainer on a shared tensor follows the synchronous one on a tiny problem."""
import torch

import sharedtensor
from sharedtensor_b200.models import GPT2, CharRNN, GPT2Config
from sharedtensor_b200.parallel.trainers import AsyncTrainer, SyncTrainer, random_token_batches


def _structured_batches(vocab, batch, seq, seed):
    """Learnable synthetic data: the next token is (token + 1) mod vocab."""
    g = torch.Generator().manual_seed(seed)
    while True:
        start = torch.randint(0, vocab, (batch, 1), generator=g)
        x = (start + torch.arange(seq + 1)) % vocab
        yield x[:, :-1].contiguous(), x[:, 1:].contiguous()


def test_char_rnn_async_matches_sync_on_one_replica(free_port):
    torch.manual_seed(0)
    m1 = CharRNN(vocab=17, hidden=32, layers=2)
    m2 = CharRNN(vocab=17, hidden=32, layers=2)
    m2.load_state_dict(m1.state_dict())
    sync = SyncTrainer(m1, lr=0.5)
    probe = CharRNN(vocab=17, hidden=32, layers=2)
    probe.load_state_dict(m2.state_dict())
    from sharedtensor_b200.models import flatten_parameters

    init, _ = flatten_parameters(probe, align=32)
    shared = sharedtensor.createOrFetch("127.0.0.1", free_port, init)
    try:
        asyn = AsyncTrainer(m2, shared, lr=0.5)
        l1 = sync.run(_structured_batches(17, 8, 12, 1), steps=60, log_every=59)
        l2 = asyn.run(_structured_batches(17, 8, 12, 1), steps=60, log_every=59)
        assert l1.loss[-1] < l1.loss[0]
        # one replica, same data, same SGD: the shared-tensor loop is the same optimisation
        assert abs(l1.loss[-1] - l2.loss[-1]) < 1e-3 * max(1.0, l1.loss[-1])
        assert l2.tokens == 60 * 8 * 12
    finally:
        shared.close()


def test_gpt2_tiny_forward_backward_and_parameter_count():
    cfg = GPT2Config.tiny()
    m = GPT2(cfg)
    batches = random_token_batches(cfg.vocab, 2, 16, torch.device("cpu"), 0)
    x, y = next(batches)
    loss = m.loss(x, y)
    loss.backward()
    assert torch.isfinite(loss)
    assert abs(float(loss) - torch.log(torch.tensor(float(cfg.vocab)))) < 1.0
    full = GPT2Config()
    n = (full.vocab + full.ctx) * full.d_model + full.n_layer * (12 * full.d_model ** 2 + 13 * full.d_model) + 2 * full.d_model
    assert n == 124_439_808
