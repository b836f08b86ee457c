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
