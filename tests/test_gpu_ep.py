"""Expert-parallel forward on one GPU: several layer shards live in one process and are stepped
phase by phase (kernels that wait on one another are never queued behind each other), so every
exchange kernel -- histogram publish, plan, row push, result push, combine -- runs for real with
"peer" buffers that are simply the other shards' buffers.

Expected: each home rank's rows equal the single-shard layer's rows bit for bit (a route's
arithmetic does not depend on where it runs, and the combine order is fixed), and match the
CPU oracle within the layer tolerance.
"""
import numpy as np
import pytest
import torch

from oracle import glmrt_oracle as O

pytestmark = pytest.mark.gpu


def to_dev(bits):
    return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).cuda()


def to_bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


@pytest.fixture(scope="module")
def small_layer():
    return O.make_layer(21, 512, 256, 16)


@pytest.mark.parametrize("world,T,max_tokens", [(2, 24, 512), (4, 30, 512), (2, 1, 512), (4, 300, 512),
                                                (2, 24, 256), (4, 7, 64), (2, 200, 256)])
def test_ep_shards_in_one_process_match_single_shard_and_oracle(pkg, small_layer, world, T, max_tokens):
    """max_tokens above 256 selects the 128-slot work items (prefill kernels) for the exchange,
    at most 256 the 32-slot ones (decode kernels); T=200 gives every expert several of those."""
    from glmrt_b200 import ep as EP
    from glmrt_b200.layer import MoeLayer
    K = 4
    hid = O.make_hidden(400 + T, T, 512)
    x = to_dev(hid)
    single = MoeLayer(512, 256, 16, K, max_tokens=512, engine="tc-ordered")   # the exchange keeps one row per route
    single.load_quantized_layer(small_layer)
    ref = to_bits(single.forward(x)).copy()
    single.check()
    single.close()

    shards = []
    for r in range(world):
        l = MoeLayer(512, 256, 16, K, max_tokens=max_tokens, ep_world=world, ep_rank=r)
        l.load_quantized_layer(small_layer)
        shards.append(l)
    EP.attach_in_process(shards)
    parts = [EP.partition_rows(T, world, r) for r in range(world)]
    assert sum(n for _, n in parts) == T
    ins = [x[s:s + n].contiguous() for s, n in parts]
    outs = [torch.zeros_like(i) for i in ins]
    for step in range(2):   # twice: epochs advance, buffers are reused
        for phase in range(4):
            for r in range(world):
                EP.forward_ep_phase(shards[r], phase, ins[r], outs[r])
            torch.cuda.synchronize()
        for l in shards:
            l.check()
    got = np.concatenate([to_bits(o) for o in outs if o.shape[0] > 0], axis=0)
    if T <= 128:
        np.testing.assert_array_equal(got, ref)
    else:
        # above 128 rows the single shard routes with the tiled logits kernel while each rank's
        # 75 rows use the decode kernel: route weights may differ in the last float32 bit
        assert O.rel_l2_per_token(got, ref).max() < 5e-3
    _, _, oo = O.layer_forward(small_layer, hid, K, mode="O1")
    assert O.rel_l2_per_token(got, oo).max() <= 2e-2
    # every rank derived the same slot layout: slots used by an owner = sum over ranks, padded per expert
    tot_routes = sum(int(l.stats().slots) for l in shards)
    assert tot_routes >= T * K
    for l in shards:
        l.close()


def test_ep_wait_that_never_completes_is_reported_not_hung(pkg, small_layer):
    """Failure detection without a GPU fault: a shard whose peer never publishes its histogram
    gives up after the bounded wait and reports it through the status channel."""
    from glmrt_b200 import ep as EP
    from glmrt_b200.layer import MoeLayer
    from glmrt_b200.native import GlmrtError
    K = 4
    shards = []
    for r in range(2):
        l = MoeLayer(512, 256, 16, K, max_tokens=64, ep_world=2, ep_rank=r)
        l.load_quantized_layer(small_layer)
        shards.append(l)
    EP.attach_in_process(shards)
    x = to_dev(O.make_hidden(1, 8, 512))
    out = torch.zeros_like(x)
    EP.forward_ep_phase(shards[0], 0, x, out)      # rank 1 never runs phase 0
    EP.forward_ep_phase(shards[0], 1, x, out)      # waits for rank 1's histogram: bounded (about 2 s)
    torch.cuda.synchronize()
    with pytest.raises(GlmrtError) as ei:
        shards[0].check()
    assert "bounded wait" in str(ei.value)
    assert shards[0].stats().chunks == 0
    for l in shards:
        l.close()


def test_ep_across_real_gpus_when_more_than_one_is_visible(pkg):
    """One process per GPU over CUDA IPC + NVLink peer stores; skipped on single-GPU boxes."""
    import os
    import subprocess
    import sys
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 2 if n < 4 else 4
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = os.path.join(root, "tests", "ep_selfcheck.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", script],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert f"EP_SELFCHECK_OK world={world}" in r.stdout


def test_a_rank_without_a_plan_poisons_its_push_and_owners_run_nothing(pkg, small_layer):
    """Rank 0 gives up waiting for rank 2's histogram (bounded wait, about 2 s) and therefore has no
    slot layout; ranks 1 and 2, whose plans succeed, have reserved slots for rank 0's routes.  Rank
    0 must say that it pushed nothing, and the owners must then run no expert work on those slots
    (no result row is stored anywhere) and report the step as failed."""
    from glmrt_b200 import ep as EP
    from glmrt_b200.layer import MoeLayer
    from glmrt_b200.native import GlmrtError
    K, world = 4, 3
    shards = []
    for r in range(world):
        l = MoeLayer(512, 256, 16, K, max_tokens=64, ep_world=world, ep_rank=r)
        l.load_quantized_layer(small_layer)
        shards.append(l)
    EP.attach_in_process(shards)
    x = to_dev(O.make_hidden(2, 30, 512))
    parts = [EP.partition_rows(30, world, r) for r in range(world)]
    ins = [x[s:s + n].contiguous() for s, n in parts]
    outs = [torch.zeros_like(i) for i in ins]
    # one good step first, so that stale destinations of an earlier step exist
    for phase in range(4):
        for r in range(world):
            EP.forward_ep_phase(shards[r], phase, ins[r], outs[r])
        torch.cuda.synchronize()
    for l in shards:
        l.check()
    before = [l.debug("ROUTE_ROWS", np.uint16).copy() for l in shards]
    # the failing step
    EP.forward_ep_phase(shards[0], 0, ins[0], outs[0])
    EP.forward_ep_phase(shards[1], 0, ins[1], outs[1])
    EP.forward_ep_phase(shards[0], 1, ins[0], outs[0])     # rank 2 has not published: expires, poisons
    torch.cuda.synchronize()
    EP.forward_ep_phase(shards[2], 0, ins[2], outs[2])     # late
    for r in (1, 2):
        EP.forward_ep_phase(shards[r], 1, ins[r], outs[r])
    torch.cuda.synchronize()
    for r in (1, 2):
        EP.forward_ep_phase(shards[r], 2, ins[r], outs[r])
    torch.cuda.synchronize()
    with pytest.raises(GlmrtError) as e0:
        shards[0].check()
    assert "bounded wait" in str(e0.value)
    for r in (1, 2):
        with pytest.raises(GlmrtError) as ei:
            shards[r].check()
        assert "no valid plan" in str(ei.value)
    after = [l.debug("ROUTE_ROWS", np.uint16) for l in shards]
    for b, a in zip(before, after):
        np.testing.assert_array_equal(a, b)
    # the context is still usable and the next step is clean
    for phase in range(4):
        for r in range(world):
            EP.forward_ep_phase(shards[r], phase, ins[r], outs[r])
        torch.cuda.synchronize()
    for l in shards:
        l.check()
    _, _, oo = O.layer_forward(small_layer, O.make_hidden(2, 30, 512), K, mode="O1")
    got = np.concatenate([to_bits(o) for o in outs], axis=0)
    assert O.rel_l2_per_token(got, oo).max() <= 2e-2
    for l in shards:
        l.close()
