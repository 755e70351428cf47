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


def test_structured_batches_follow_their_rule():
    """Token t+1 = (token t + step) mod m with one step per sequence; a large vocabulary is narrowed to m active
    tokens, a small one is used whole."""
    from sharedtensor_b200.parallel.trainers import structured_token_batches

    for vocab, m in ((13, 13), (50257, 512)):
        x, y = next(structured_token_batches(vocab, 6, 20, torch.device("cpu"), seed=3, period=7))
        assert x.shape == (6, 20) and y.shape == (6, 20)
        assert int(x.max()) < m and int(y.max()) < m and int(x.min()) >= 0
        assert torch.equal(x[:, 1:], y[:, :-1])
        step = (y - x) % m
        assert bool((step == step[:, :1]).all()) and 1 <= int(step.min()) and int(step.max()) <= 7


def test_two_async_replicas_learn_together(free_port):
    """Two replicas train on different shards of a learnable task through one shared tensor; both losses fall and
    the replicas end up with the same parameters."""
    import threading

    from sharedtensor_b200.models import flatten_parameters
    from sharedtensor_b200.parallel.trainers import structured_token_batches

    torch.manual_seed(1)
    models = [CharRNN(vocab=13, hidden=24, layers=1) for _ in range(2)]
    models[1].load_state_dict(models[0].state_dict())
    init, _ = flatten_parameters(models[0], align=32)
    shared = [sharedtensor.createOrFetch("127.0.0.1", free_port, init.clone()) for _ in range(2)]
    logs = [None, None]

    def work(i):
        tr = AsyncTrainer(models[i], shared[i], lr=0.3)
        data = structured_token_batches(13, 8, 10, torch.device("cpu"), seed=10 + i, period=1)
        logs[i] = tr.run(data, steps=120, log_every=119)

    try:
        ts = [threading.Thread(target=work, args=(i,)) for i in range(2)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        for lg in logs:
            assert lg.loss[-1] < 0.9 * lg.loss[0], (lg.loss[0], lg.loss[-1])
        a, b = torch.empty_like(init), torch.empty_like(init)

        def agree():
            shared[0].copyToTensor(a)
            shared[1].copyToTensor(b)
            return float((a - b).norm() / a.norm()) < 1e-3

        import time

        deadline = time.time() + 20
        while time.time() < deadline and not agree():
            time.sleep(0.05)
        assert agree()
    finally:
        for s in reversed(shared):
            s.close()
