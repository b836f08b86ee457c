"""GPU parity for the greedy token pick, through the C-ABI (zen_cuda_dev_greedy_pick).

Bar: the picked index is identical to the oracle's restatement of the reference's greedy rule
(sample_logits, src/adapters/dense_transformer_runtime.cpp:391-418): first maximum among the finite logits,
-1 when there is none.
"""
import numpy as np
import pytest

from zeninfer_b200 import shard

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from zeninfer_b200 import Backend
    return Backend()


def gpu_pick(be, logits: np.ndarray, cuts=None) -> np.ndarray:
    """logits [tokens, vocab]; cuts: shard boundaries, which lays the row out as the gathered shards of a sharded
    lm_head: [shard][token][shard rows], every shard padded to the widest."""
    import torch
    tokens, vocab = logits.shape
    pick = torch.full((tokens,), 12345, dtype=torch.int64, device="cuda")
    if cuts is None:
        d = torch.from_numpy(np.ascontiguousarray(logits)).cuda()
        segs = [(d.data_ptr(), vocab, 0, vocab)]
    else:
        widest = max(b - a for a, b in cuts)
        slot = tokens * widest
        host = np.full((len(cuts), slot), np.nan, np.float32)  # padding that would win nothing and must not be read
        for r, (a, b) in enumerate(cuts):
            host[r, : tokens * (b - a)] = logits[:, a:b].reshape(-1)
        d = torch.from_numpy(host).cuda()
        segs = [(d.data_ptr() + 4 * r * slot, b - a, a, b - a) for r, (a, b) in enumerate(cuts)]
    be.dev_greedy_pick(segs, tokens, pick.data_ptr(), 0)
    torch.cuda.synchronize()
    be.dev_check(0)
    return pick.cpu().numpy()


def oracle_pick(zo, logits: np.ndarray) -> np.ndarray:
    return np.array([zo.argmax(row) for row in logits], np.int64)


@pytest.mark.parametrize("tokens,vocab", [(1, 1), (1, 31), (3, 4097), (8, 128256)])
def test_random_logits(be, zo, tokens, vocab):
    logits = np.random.default_rng(vocab + tokens).standard_normal((tokens, vocab), dtype=np.float32)
    assert np.array_equal(gpu_pick(be, logits), oracle_pick(zo, logits))


def test_ties_go_to_the_lowest_index_and_zeros_are_equal(be, zo):
    rng = np.random.default_rng(7)
    logits = np.round(rng.standard_normal((8, 50000), dtype=np.float32) * 2)  # few distinct values: many ties at the maximum
    logits[0, :] = 0.0
    logits[0, 0] = -0.0      # -0.0 equals +0.0: index 0 must win
    logits[1, :] = -3.0
    logits[1, 40000] = -0.0
    logits[1, 45000] = 0.0
    assert np.array_equal(gpu_pick(be, logits), oracle_pick(zo, logits))


def test_non_finite_logits_never_win(be, zo):
    rng = np.random.default_rng(11)
    logits = rng.standard_normal((6, 20000), dtype=np.float32)
    logits[0, 5] = np.inf
    logits[1, 17] = np.nan
    logits[2, :] = np.nan                  # no candidate at all
    logits[3, :] = -np.inf
    logits[3, 19999] = -3.0e38             # the only finite entry, and the most negative one possible
    logits[4, ::2] = np.inf
    logits[5, :] = np.float32(-3.4e38)
    got = gpu_pick(be, logits)
    assert np.array_equal(got, oracle_pick(zo, logits))
    assert got[2] == -1 and got[3] == 19999 and got[5] == 0


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("tokens", [1, 8])
def test_gathered_shard_layout(be, zo, world, tokens):
    vocab = 128256
    logits = np.random.default_rng(world * 10 + tokens).standard_normal((tokens, vocab), dtype=np.float32)
    logits[0, 100] = logits[0].max() + 1      # maximum in the first shard
    if tokens > 1:
        top = logits[1].max() + 1
        a, b = shard.shard_plan(vocab, world)[-1]
        logits[1, a] = top                    # the same maximum in the last shard and in the first:
        logits[1, 3] = top                    # the lower index wins
    assert np.array_equal(gpu_pick(be, logits, shard.shard_plan(vocab, world)), oracle_pick(zo, logits))


def test_bad_arguments_are_errors(be):
    from zeninfer_b200.backend import BackendError
    with pytest.raises(BackendError):
        be.dev_greedy_pick([(0, 16, 0, 16)], 1, 0, 0)          # null output
    with pytest.raises(BackendError):
        be.dev_greedy_pick([], 1, 1, 0)                        # no segment


# ---- temperature / top-k / top-p sampling (zen_cuda_dev_sample) against a numpy restatement of sampling_distribution ----
def reference_distribution(logits: np.ndarray, temperature: float, top_k: int, top_p: float) -> np.ndarray:
    """sampling_distribution (src/adapters/dense_transformer_runtime.cpp:349-383) restated: probabilities by token id."""
    temperature = float(np.float32(temperature))     # GenerationOptions::temperature is a float, promoted in the division
    prob = np.zeros(logits.size, np.float64)
    order = np.flatnonzero(np.isfinite(logits))
    if order.size == 0:
        return prob
    order = order[np.argsort(-logits[order].astype(np.float64), kind="stable")]      # by value, equal values by id
    if top_k and top_k < order.size:
        order = order[:top_k]
    p = np.exp((logits[order].astype(np.float64) - float(logits[order[0]])) / temperature)
    p /= p.sum()
    if 0.0 < top_p < 1.0:
        cum = np.cumsum(p)
        keep = int(np.argmax(cum >= top_p)) + 1 if (cum >= top_p).any() else order.size
        order, p = order[:max(1, keep)], p[:max(1, keep)]
        p = p / p.sum()
    prob[order] = p
    return prob


@pytest.mark.parametrize("n,temperature,top_k,top_p", [(128256, 0.8, 40, 0.95), (128256, 1.0, 50, 1.0), (128256, 0.7, 0, 0.9), (5000, 1.3, 1024, 0.5),
                                                      (300, 0.5, 1000, 0.99), (128256, 0.25, 1, 1.0), (1031, 2.0, 7, 0.3)])
def test_sampling_matches_the_reference_distribution(be, n, temperature, top_k, top_p):
    import torch
    rng = np.random.default_rng(n + top_k)
    logits = (rng.standard_normal(n) * 2.0).astype(np.float32)
    logits[rng.integers(0, n, size=5)] = np.float32("nan")
    logits[rng.integers(0, n, size=3)] = np.float32("inf")       # non-finite logits never enter the distribution
    want = reference_distribution(logits, temperature, top_k, top_p)
    fits = np.count_nonzero(want) <= 1024          # else the device keeps the 1024 most likely tokens and says so
    if not fits:
        finite = np.flatnonzero(np.isfinite(logits))
        top = finite[np.argsort(-logits[finite].astype(np.float64), kind="stable")][:1024]
        want = np.zeros_like(want)
        want[top] = np.exp((logits[top].astype(np.float64) - float(logits[top[0]])) / float(np.float32(temperature)))
        want /= want.sum()
    d_logits = torch.from_numpy(logits).cuda()
    d_pick = torch.full((1,), -7, dtype=torch.int64, device="cuda")
    d_ids = torch.full((1024,), -1, dtype=torch.int32, device="cuda")
    d_probs = torch.zeros(1024, dtype=torch.float64, device="cuda")
    d_count = torch.zeros(1, dtype=torch.int32, device="cuda")
    d_trunc = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    kept = np.flatnonzero(want)
    cum = np.cumsum(want[kept])
    for u in (0.0, 0.25, 0.5, 0.999999, float(rng.random()), float(rng.random())):
        be.dev_sample(d_logits.data_ptr(), n, temperature, top_k, top_p, u, d_pick.data_ptr(), 0, d_kept_ids=d_ids.data_ptr(),
                      d_kept_probs=d_probs.data_ptr(), d_kept_count=d_count.data_ptr(), d_truncated=d_trunc.data_ptr())
        torch.cuda.synchronize()
        be.dev_check(0)
        count = int(d_count.item())
        assert count == kept.size
        assert d_ids[:count].cpu().tolist() == kept.tolist()                       # the kept set, in ascending token id
        assert np.allclose(d_probs[:count].cpu().numpy(), want[kept], rtol=1e-12, atol=1e-15)
        expect = kept[min(int(np.searchsorted(cum, u, side="left")), kept.size - 1)]   # first cumulative >= u, in token-id order
        got = int(d_pick.item())
        if got != expect:     # only a u within rounding of a cumulative boundary may land on the neighbour
            j = int(np.searchsorted(kept, got))
            assert abs(cum[j] - u) < 1e-9 or (j and abs(cum[j - 1] - u) < 1e-9), (u, got, expect)
        assert int(d_trunc.item()) == (0 if fits else 1)


def test_sampling_ties_and_degenerate_rows(be):
    import torch
    # all logits equal: top_k = 5 keeps the five lowest ids with equal probabilities
    d_logits = torch.full((5000,), 1.5, device="cuda")
    d_pick = torch.zeros(1, dtype=torch.int64, device="cuda")
    d_ids = torch.full((1024,), -1, dtype=torch.int32, device="cuda")
    d_probs = torch.zeros(1024, dtype=torch.float64, device="cuda")
    d_count = torch.zeros(1, dtype=torch.int32, device="cuda")
    be.dev_sample(d_logits.data_ptr(), 5000, 1.0, 5, 1.0, 0.55, d_pick.data_ptr(), 0, d_kept_ids=d_ids.data_ptr(), d_kept_probs=d_probs.data_ptr(), d_kept_count=d_count.data_ptr())
    torch.cuda.synchronize()
    assert int(d_count.item()) == 5 and d_ids[:5].cpu().tolist() == [0, 1, 2, 3, 4]
    assert np.allclose(d_probs[:5].cpu().numpy(), 0.2) and int(d_pick.item()) == 2        # cumulative 0.2, 0.4, 0.6: u = 0.55 -> id 2
    # no finite logit: -1, nothing kept
    d_bad = torch.full((100,), float("nan"), device="cuda")
    be.dev_sample(d_bad.data_ptr(), 100, 1.0, 0, 1.0, 0.5, d_pick.data_ptr(), 0, d_kept_count=d_count.data_ptr())
    torch.cuda.synchronize()
    assert int(d_pick.item()) == -1 and int(d_count.item()) == 0
    # a flat distribution without a top-k cut: the 1024-candidate limit is reported
    d_flat = torch.zeros(4000, device="cuda")
    d_trunc = torch.zeros(1, dtype=torch.int32, device="cuda")
    be.dev_sample(d_flat.data_ptr(), 4000, 1.0, 0, 0.9, 0.5, d_pick.data_ptr(), 0, d_kept_count=d_count.data_ptr(), d_truncated=d_trunc.data_ptr())
    torch.cuda.synchronize()
    assert int(d_trunc.item()) == 1 and int(d_count.item()) == 1024     # the 1024 candidates hold 0.256 of the mass: short of 0.9
    from zeninfer_b200 import BackendError
    with pytest.raises(BackendError):
        be.dev_sample(d_flat.data_ptr(), 4000, 0.0, 0, 0.9, 0.5, d_pick.data_ptr(), 0)     # temperature must be positive
