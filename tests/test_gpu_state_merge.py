"""GPU parity of the public state-merge operator against the CPU oracle's split-K merge
(single_decode_bf16_split_k_merge_reference, crates/loom-infer/src/attention/single_decode/
mod.rs:343-379), through the C ABI.  Tolerances are the decode gates': O max-abs 2e-2 and
row-relative 1e-2, LSE 1e-3 (log2)."""
import numpy as np
import pytest
import torch

import loom_kernels_b200 as lk
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def provider():
    return lk.DecodeProvider.load(0)


def random_states(rng, rows, partitions, empty_fraction=0.0):
    """Plausible partial states: max_log2 ~ N(0, 3), normaliser in [1, 16], wv = normaliser *
    (a convex-ish mix of N(0,1) rows).  Some states are empty ([0, 0, 0...])."""
    states = np.zeros((rows, partitions, 130), dtype=np.float32)
    states[:, :, 0] = rng.normal(0.0, 3.0, size=(rows, partitions))
    states[:, :, 1] = rng.uniform(1.0, 16.0, size=(rows, partitions))
    states[:, :, 2:] = rng.standard_normal((rows, partitions, 128)) * states[:, :, 1:2]
    empty = rng.random((rows, partitions)) < empty_fraction
    empty[:, 0] = False  # keep one state per row
    states[empty] = 0.0
    return states


def merge_on_gpu(provider, states, sentinel=float("nan")):
    rows, partitions, _ = states.shape
    plan = provider.plan_state_merge(rows, partitions)
    queue = lk.CommandQueue(torch.cuda.Stream(), 1)
    dev_states = torch.from_numpy(states.reshape(-1)).to("cuda:0")
    out = torch.full((rows * 128,), sentinel, dtype=torch.bfloat16, device="cuda:0")
    lse = torch.full((rows,), sentinel, dtype=torch.float32, device="cuda:0")
    torch.cuda.synchronize()
    b = queue.bindings(3)
    hs, ho, hl = b.bind_read(dev_states), b.bind_read_write(out), b.bind_read_write(lse)
    scope = queue.begin(b)
    plan.enqueue_into(scope, lk.StateMergeArgs(hs, ho.write(), hl.write()))
    b = scope.finish().wait()
    return H.host_bits(b.take_read_write(ho)), b.take_read_write(hl).cpu().numpy()


@pytest.mark.parametrize("rows,partitions,empty", [(1, 1, 0.0), (32, 8, 0.0), (64, 16, 0.3),
                                                   (5, 100, 0.5), (2048, 3, 0.0)])
def test_merge_matches_the_cpu_reference(provider, oracle, rows, partitions, empty):
    states = random_states(np.random.default_rng(rows * 131 + partitions), rows, partitions, empty)
    expected_out, expected_lse = oracle.split_k_merge(rows, partitions, states.reshape(-1))
    out, lse = merge_on_gpu(provider, states)
    e, a = H.bits_to_f32(expected_out).reshape(rows, 128), H.bits_to_f32(out).reshape(rows, 128)
    assert np.all(np.isfinite(a))
    assert np.abs(a - e).max() <= 2e-2
    rel = np.linalg.norm(a - e, axis=1) / np.maximum(np.linalg.norm(e, axis=1), 1e-6)
    assert rel.max() <= 1e-2
    assert np.abs(lse - expected_lse).max() <= 1e-3


def test_rows_without_any_state_stay_unwritten(provider):
    states = random_states(np.random.default_rng(7), 4, 3)
    states[2] = 0.0  # every state of row 2 is empty
    out, lse = merge_on_gpu(provider, states, sentinel=-7.0)
    sentinel = H.host_bits(torch.tensor([-7.0], dtype=torch.bfloat16))[0]
    assert np.all(out[2 * 128:3 * 128] == sentinel) and lse[2] == -7.0
    assert np.all(out[:2 * 128] != sentinel) and np.all(lse[[0, 1, 3]] != -7.0)
