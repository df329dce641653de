"""The sampler: host semantics (no GPU) and host/device agreement (GPU)."""
import numpy as np
import pytest
import torch

from ember_b200.sampling import SamplingParams, gumbel_noise, sample_host, sampling_distribution


def test_host_greedy_and_top_k_one():
    l = np.array([0.1, 3.0, 3.0, -1.0], dtype=np.float32)
    assert sample_host(l, SamplingParams(temperature=0.0), 5) == 1            # lowest index on ties
    assert sample_host(l, SamplingParams(temperature=1.0, top_k=1, seed=3), 5) == 1


def test_host_filters():
    l = np.log(np.array([0.5, 0.25, 0.125, 0.0625, 0.0625], dtype=np.float64)).astype(np.float32)
    d = sampling_distribution(l, SamplingParams(temperature=1.0, top_p=0.8))
    assert [t for t, _ in d] == [0, 1, 2]                                     # 0.5 + 0.25 + 0.125 >= 0.8
    d = sampling_distribution(l, SamplingParams(temperature=1.0, min_p=0.3))
    assert [t for t, _ in d] == [0, 1]                                        # p >= 0.3 * 0.5
    d = sampling_distribution(l, SamplingParams(temperature=1.0, top_k=4, top_p=0.99))
    assert [t for t, _ in d] == [0, 1, 2, 3] and abs(sum(p for _, p in d) - 1.0) < 1e-6


def test_host_noise_is_stateless():
    assert gumbel_noise(7, 11, 13) == gumbel_noise(7, 11, 13)
    assert gumbel_noise(7, 11, 13) != gumbel_noise(7, 12, 13)
    g = np.array([gumbel_noise(1, c, 0) for c in range(4000)], dtype=np.float64)
    assert abs(g.mean() - 0.5772) < 0.06                                      # Gumbel(0, 1) mean


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [1000, 4099, 151936])
def test_device_equals_host(vocab):
    from ember_b200.sampling import device
    rng = np.random.default_rng(vocab)
    rows = 24
    logits = (rng.normal(size=(rows, vocab)) * 2.5).astype(np.float32)
    logits[3, 10] = logits[3, 500] = logits[3].max() + 1.0                      # a tie at the top
    logits[5, :] = np.round(logits[5, :])                                       # many ties everywhere
    variants = [SamplingParams(temperature=0.0), SamplingParams(temperature=0.8, top_k=40, top_p=0.9, seed=11),
                SamplingParams(temperature=1.3, top_p=0.7, seed=12), SamplingParams(temperature=0.6, top_k=5, seed=13),
                SamplingParams(temperature=1.0, min_p=0.05, seed=14), SamplingParams(temperature=1.0, seed=15),
                SamplingParams(temperature=0.9, top_k=20, top_p=0.8, min_p=0.02, seed=16),
                SamplingParams(temperature=1.0, top_k=1, seed=17)]
    params = [variants[r % len(variants)] for r in range(rows)]
    counters = [100 + 3 * r for r in range(rows)]
    got = device.sample(torch.from_numpy(logits).cuda(), params, counters).cpu().tolist()
    want = [sample_host(logits[r], params[r], counters[r]) for r in range(rows)]
    assert got == want


@pytest.mark.gpu
@pytest.mark.parametrize("vocab", [17, 1000, 151936])
def test_device_greedy_rows_take_the_lowest_index_on_ties(vocab):
    from ember_b200.sampling import device
    rng = np.random.default_rng(vocab)
    logits = rng.normal(size=(9, vocab)).astype(np.float32)
    logits[2, [3, vocab - 1]] = 50.0                   # a tie far apart
    logits[4, :] = 1.0                                 # everything ties: index 0
    logits[6, vocab - 1] = 99.0                        # the very last entry
    got = device.sample(torch.from_numpy(logits).cuda(), [SamplingParams(temperature=0.0)] * 9, [0] * 9).cpu().tolist()
    assert got == [int(np.argmax(r)) for r in logits]


@pytest.mark.gpu
def test_device_draws_stay_in_the_kept_set_and_follow_the_distribution():
    from ember_b200.sampling import device
    rng = np.random.default_rng(5)
    vocab, draws = 2000, 2000
    row = (rng.normal(size=vocab) * 3).astype(np.float32)
    p = SamplingParams(temperature=0.8, top_k=40, top_p=0.9, seed=77)
    dist = dict(sampling_distribution(row, p))
    logits = torch.from_numpy(np.tile(row, (draws, 1))).cuda()
    got = device.sample(logits, [p] * draws, list(range(draws))).cpu().numpy()
    assert set(got.tolist()) <= set(dist)
    top = max(dist, key=dist.get)
    freq, pt = float((got == top).mean()), dist[top]
    assert abs(freq - pt) < 4 * np.sqrt(pt * (1 - pt) / draws)
