"""GPU parity of top-k selection and the on-device samplers against the oracle's restatement of
models/kalosm-llama/src/sampler.rs, on identical logits, previous tokens and draws."""
import numpy as np
import pytest

import fixtures as F
import kalosm_b200 as kb
from gpu_util import dev  # noqa: F401
from llama_util import build_models, tiny_cfg
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_top_k_pairs(dev):
    # Tensor::top_k_pairs (fusor-ml/fusor/src/lib.rs:416-453): descending, ties -> higher id, non-finite skipped
    rng = np.random.default_rng(1)
    logits = rng.standard_normal((5, 128256)).astype(np.float32)
    logits[1, rng.choice(128256, 3000, replace=False)] = 2.5     # many equal values around the cut
    logits[2, :] = -1.0                                           # everything ties
    logits[3, rng.choice(128256, 500, replace=False)] = np.nan
    logits[3, rng.choice(128256, 500, replace=False)] = np.inf
    logits[3, rng.choice(128256, 500, replace=False)] = -np.inf
    logits[4, :] = np.nan
    logits[4, [7, 99]] = [0.5, 0.5]                               # fewer finite values than k
    t = dev.tensor(logits)
    for k in (1, 2, 5, 64, 1000, 1024):
        ids, vals = dev.top_k(t, k)
        ids, vals = ids.as_slice(), vals.as_slice()
        for r in range(5):
            oid, oval = O.top_k(logits[r], k)
            assert np.array_equal(ids[r, :len(oid)], oid), (k, r)
            assert np.array_equal(vals[r, :len(oid)], oval), (k, r)
            assert np.all(ids[r, len(oid):] == 0xFFFFFFFF) and np.all(np.isneginf(vals[r, len(oid):]))
    small = rng.standard_normal((3, 50)).astype(np.float32)
    ids, vals = dev.top_k(dev.tensor(small), 64)
    for r in range(3):
        oid, oval = O.top_k(small[r], 64)
        assert len(oid) == 50 and np.array_equal(ids.as_slice()[r, :50], oid)
    with pytest.raises(kb.FusorError) as e:
        dev.top_k(t, 1025)
    assert e.value.code == kb.ERR_INVALID_ARGUMENT


CONFIGS = [
    dict(temperature=1.0, top_k=4),
    dict(temperature=0.8, top_k=40, top_p=0.9),
    dict(temperature=1.3, top_k=64, min_p=0.05),
    dict(temperature=0.7, top_k=50, top_p=0.95, min_p=0.02, repetition_penalty=1.3, repetition_penalty_range=48),
    dict(temperature=0.0, top_k=8, repetition_penalty=1.5, repetition_penalty_range=200),
    dict(temperature=1.0, top_k=1024, top_p=0.999),
]


@pytest.mark.parametrize("cfg", CONFIGS, ids=lambda c: "-".join(f"{k[:5]}{v}" for k, v in c.items()))
def test_standard_sampler_matches_the_oracle(dev, cfg):
    rng = np.random.default_rng(11)
    rows, n = 3, 32000
    logits = (3.0 * rng.standard_normal((rows, n))).astype(np.float32)
    logits[0, 5] = np.nan
    logits[1, 9] = np.inf
    prev = rng.integers(0, n, size=(rows, 120), dtype=np.uint32)
    prev[:, -10:] = np.argsort(-np.nan_to_num(logits, nan=-1e9, posinf=-1e9), axis=1)[:, :10]  # penalise the leaders
    t, pv = dev.tensor(logits), dev.tensor(prev)
    decided = 0
    for seed in range(6):
        for counter in (0, 1, 77):
            c = kb.SamplerConfig(seed=seed, **cfg)
            got = dev.sample(t, c, previous=pv, counter=counter).as_slice()
            for r in range(rows):
                want, margin, _ = O.sample(logits[r], previous=prev[r], seed=seed, counter=counter, row=r, **cfg)
                if margin > 1e-5:  # otherwise one ulp of an exponential decides
                    assert got[r] == want, (cfg, seed, counter, r, margin)
                    decided += 1
    assert decided >= 18  # a third of the draws at least are clear of every boundary (1024 candidates leave few)


def test_sampler_distribution_properties(dev):
    # the reference's own sampler tests (models/kalosm-llama/src/sampler.rs:372-441) on the device:
    # flat logits reach past the first candidate; top-p 0.5 keeps two of four; min-p keeps the leader
    flat = dev.tensor(np.zeros((1, 4), np.float32))
    seen = {int(dev.sample(flat, kb.SamplerConfig(top_k=4, seed=s)).as_slice()[0]) for s in range(64)}
    assert seen - {3}
    seen = {int(dev.sample(flat, kb.SamplerConfig(top_k=4, top_p=0.5, seed=s)).as_slice()[0]) for s in range(64)}
    assert seen <= {2, 3} and seen
    steep = dev.tensor(np.array([[-5.0, -4.0, -3.0, 0.0]], np.float32))
    assert int(dev.sample(steep, kb.SamplerConfig(top_k=4, min_p=0.1, seed=0)).as_slice()[0]) == 3
    seen = {int(dev.sample(flat, kb.SamplerConfig(strategy=kb.SAMPLER_MIROSTAT2, top_k=4, seed=s),
                           mu=dev.tensor(np.array([10.0], np.float32))).as_slice()[0]) for s in range(64)}
    assert seen - {3}
    empty = dev.tensor(np.full((1, 16), np.nan, np.float32))
    assert int(dev.sample(empty, kb.SamplerConfig(top_k=4)).as_slice()[0]) == 0xFFFFFFFF


def test_mirostat2_matches_the_oracle(dev):
    rng = np.random.default_rng(21)
    n = 5000
    for seed in range(4):
        mu_cpu = 6.0
        mu_gpu = dev.tensor(np.array([mu_cpu], np.float32))
        for step in range(12):
            logits = (2.5 * rng.standard_normal((1, n))).astype(np.float32)
            cfg = dict(strategy=1, temperature=0.9, top_k=32, tau=4.0, eta=0.2)
            got = dev.sample(dev.tensor(logits), kb.SamplerConfig(seed=seed, mu=mu_cpu, **cfg), counter=step,
                             mu=mu_gpu).as_slice()[0]
            want, margin, mu_cpu = O.sample(logits[0], seed=seed, counter=step, mu=mu_cpu, **cfg)
            if margin <= 1e-5:
                break
            assert got == want, (seed, step, margin)
            assert abs(mu_gpu.as_slice()[0] - mu_cpu) < 1e-4


@pytest.mark.parametrize("batch", [1, 2])
def test_generate_sampled_matches_stepwise_oracle(dev, batch):
    # The device-resident sampled loop (fused step or captured graph + sampler kernel per step,
    # nothing read back in between). Its tokens are replayed through forward() on the same model
    # (the same kernels, so the same logits bit for bit) and every draw is repeated by the oracle's
    # sampler on those logits with the session's history as penalty window and the position as
    # draw counter. Logit parity with the oracle's forward pass is the subject of test_gpu_llama.
    cfg = tiny_cfg()
    gpu, cpu = build_models(dev, cfg, batch=batch, seed=41)
    rng = np.random.default_rng(42)
    prompt = rng.integers(0, cfg["vocab"], size=(batch, 6), dtype=np.uint32)
    lg, first = gpu.forward(prompt)
    assert F.rel_l2(lg, cpu.forward(prompt)) < 2e-3
    scfg = dict(temperature=0.9, top_k=30, top_p=0.95, repetition_penalty=1.2, repetition_penalty_range=16)
    steps = 12
    got = gpu.generate_sampled(first, steps, kb.SamplerConfig(seed=5, **scfg))
    assert got.shape == (batch, steps) and gpu.position == 6 + steps
    assert dev.status() == 0
    gpu.reset()
    gpu.forward(prompt)
    history = [list(prompt[b]) + [int(first[b])] for b in range(batch)]
    tok = first.copy()
    decided = 0
    for s in range(steps):
        lg, _ = gpu.forward(tok[:, None])
        for b in range(batch):
            want, margin, _ = O.sample(lg[b], previous=np.array(history[b], np.uint32), seed=5,
                                       counter=len(history[b]), row=b, **scfg)
            if margin > 1e-5:  # otherwise one ulp of an exponential decides
                assert got[b, s] == want, (b, s, margin)
                decided += 1
            history[b].append(int(got[b, s]))
            tok[b] = got[b, s]
    assert decided >= steps * batch // 2
    # the samplers do not disturb greedy decoding afterwards: temperature 0 = greedy ids
    gpu.reset()
    _, first = gpu.forward(prompt)
    greedy = gpu.generate_greedy(first, 6)
    gpu.reset()
    gpu.forward(prompt)
    assert np.array_equal(gpu.generate_sampled(first, 6, kb.SamplerConfig(temperature=0.0, top_k=5)), greedy)
