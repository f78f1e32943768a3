"""Head outputs delivered into the ranks' exchange buffers by the fused decode
kernel itself (shainet_attn_comm_*).  The one-rank case runs on any GPU box; the
two-rank case needs two GPUs and runs as two child processes, one per GPU."""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import DECODE_TOL, Q30, make_pair, qkv, rel_err
from shainet_b200 import _lib

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ctx():
    import shainet_b200 as S
    c = S.AttnContext(0)
    yield c
    c.close()


def test_self_delivery_matches_the_plain_output(ctx):
    """world = 1: the kernel stores every head row and log-sum-exp into its own
    exchange buffer at the armed offsets as {value, epoch} words, the wait kernel
    unpacks them; the values equal what the same call leaves in `out`, and the oracle."""
    import torch
    import shainet_b200 as S
    rng = np.random.default_rng(6001)
    shape = Q30
    H, hd = shape["H"], shape["hd"]
    o, g = make_pair(ctx, shape, rng, initial_capacity=4096)
    L0 = 3000
    q, k, v = qkv(rng, shape, L0)
    o.attend_cached(q, k, v, threads=8)
    g.cache.import_(*o.export_cache())
    slot = H * hd + H
    handle = ctx.comm_create(3 * slot)
    assert len(handle) == 64
    ctx.comm_open([handle], 0)
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    out = torch.empty(H * hd, device=dev)
    lse = torch.empty(H, device=dev)
    for step in range(3):
        q, k, v = qkv(rng, shape, 1)
        ref = o.attend_cached(q, k, v, threads=8)[0]
        tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (q, k, v))
        off = step * slot
        ctx.set_lse_out(lse.data_ptr())
        ctx.comm_set_target(off, off + H * hd, epoch=step + 7)
        g.forward_cached_dev(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), 1, stream=stream)
        ctx.comm_wait(off, slot, step + 7, stream)
        got = np.empty(slot, np.float32)
        ctx.comm_read(off, got, stream)
        torch.cuda.synchronize()
        ctx.sync()
        ctx.set_lse_out(None)
        assert np.array_equal(got[:H * hd], out.cpu().numpy())
        assert np.array_equal(got[H * hd:], lse.cpu().numpy())
        assert rel_err(got[:H * hd], ref) <= DECODE_TOL
    # an armed delivery that the kernel cannot do is refused, and disarmed
    q, k, v = qkv(rng, shape, 4)
    tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (q, k, v))
    out4 = torch.empty(4 * H * hd, device=dev)
    ctx.comm_set_target(0, -1, 99)
    with pytest.raises(S.ShainetAttnError) as ei:
        g.forward_cached_dev(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out4.data_ptr(), 4, stream=stream)
    assert ei.value.code == _lib.E_UNSUPPORTED
    g.forward_cached_dev(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out4.data_ptr(), 4, stream=stream)
    ctx.sync()
    ctx.comm_set_target(3 * slot, -1, 1)   # one slot past the end of the buffer
    with pytest.raises(S.ShainetAttnError) as ei:
        g.forward_cached_dev(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), 1, stream=stream)
    assert ei.value.code == _lib.E_INVALID
    g.close()


def test_wait_for_a_flag_nobody_raises_reports_a_timeout():
    """The wait for delivered words is bounded: with no producer it gives up after about a second
    and the next sync reports SHAINET_ATTN_E_DEVICE_WAIT; the context stays usable."""
    import shainet_b200 as S
    c = S.AttnContext(0)
    c.comm_open([c.comm_create(64)], 0)
    c.comm_wait(8, 16, 12345)
    with pytest.raises(S.ShainetAttnError) as ei:
        c.sync()
    assert ei.value.code == _lib.E_DEVICE_WAIT
    c.sync()
    c.close()


def test_the_cross_rank_wait_limit_is_a_context_setting():
    """A host whose ranks may be late by more (or must fail faster) than the default second sets the
    limit itself: 50 ms here, observed through the time the abandoned wait took."""
    import time
    import shainet_b200 as S
    c = S.AttnContext(0)
    c.comm_open([c.comm_create(64)], 0)
    with pytest.raises(S.ShainetAttnError) as ei:
        c.comm_set_wait_limit_ms(0)
    assert ei.value.code == _lib.E_INVALID
    c.comm_set_wait_limit_ms(50)
    c.sync()
    t0 = time.perf_counter()
    c.comm_wait(0, 16, 777)
    with pytest.raises(S.ShainetAttnError) as ei:
        c.sync()
    waited = time.perf_counter() - t0
    assert ei.value.code == _lib.E_DEVICE_WAIT
    assert 0.04 <= waited < 0.6, waited
    c.sync()
    c.close()


WORKER = r"""
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.path.join(sys.argv[1], "tests")); sys.path.insert(0, sys.argv[1])
import shainet_b200 as S
from helpers import Q30, qkv, rel_err, DECODE_TOL
from oracle import oracle as O
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo")
# "heads": two kv-head groups, one per rank.  "split": one kv head, the two ranks hold alternate positions.
shape = Q30 if sys.argv[2] == "heads" else dict(H=8, KV=1, hd=128, theta=1e6, qk_norm=True)
H, KV, hd = shape["H"], shape["KV"], shape["hd"]
sp = S.sharding.plan(world, rank, H, KV)
Hl, KVl = sp.head_count, sp.kv_count
split = sp.seq_parts > 1
rng = np.random.default_rng(6100)            # same stream on every rank: identical full inputs
qn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
kn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
o = O.OracleAttention(H, KV, hd, shape["theta"], 1e-6, q_norm=qn, k_norm=kn)
ctx = S.AttnContext(rank)
g = S.LlamaAttention(ctx, Hl, KVl, hd, shape["theta"], 1e-6, q_norm=qn, k_norm=kn, initial_capacity=4096)
L0 = 3001
q, k, v = qkv(rng, shape, L0)
o.attend_cached(q, k, v, threads=8)
kc, vc = o.export_cache()
g.cache.import_(kc[sp.kv_begin:sp.kv_begin + KVl, sp.seq_part::sp.seq_parts],
                vc[sp.kv_begin:sp.kv_begin + KVl, sp.seq_part::sp.seq_parts])
assert len(g.cache) == sp.local_rows(L0)
slots = 2
pay = Hl * hd + (Hl if split else 0)
mine = ctx.comm_create(slots * world * pay)
handles = [None] * world
dist.all_gather_object(handles, mine)
ctx.comm_open(handles, rank)
dist.barrier()
dev = torch.device("cuda", rank)
stream = torch.cuda.current_stream().cuda_stream
out = torch.empty(Hl * hd, device=dev)
merged = torch.empty(H * hd, device=dev)
worst = 0.0
for step in range(6):
    pos = L0 + step
    q, k, v = qkv(rng, shape, 1)
    ref = o.attend_cached(q, k, v, threads=8)[0]
    ql = q.reshape(1, H, hd)[:, sp.head_begin:sp.head_begin + Hl].reshape(1, -1).copy()
    kl = k.reshape(1, KV, hd)[:, sp.kv_begin:sp.kv_begin + KVl].reshape(1, -1).copy()
    vl = v.reshape(1, KV, hd)[:, sp.kv_begin:sp.kv_begin + KVl].reshape(1, -1).copy()
    tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (ql, kl, vl))
    slot = step % slots
    mine_off = (slot * world + rank) * pay
    lse_off = mine_off + Hl * hd if split else -1
    own = sp.owns_position(pos)
    if split and step % 2 == 0:   # deliver + wait + merge of the sequence parts in one call
        g.forward_cached_dev_exchange_merge(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), pos, own,
                                            slot * world * pay, sp.seq_parts, step + 1, merged.data_ptr(), stream=stream)
        torch.cuda.synchronize(); ctx.sync()
        worst = max(worst, rel_err(merged.cpu().numpy(), ref))
        dist.barrier()
        continue
    if step % 2 == 0 and not split:
        ctx.comm_set_target(mine_off, lse_off, step + 1)
        g.forward_cached_dev(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), 1, stream=stream)
        ctx.comm_wait(slot * world * pay, world * pay, step + 1, stream)
    else:   # the same three steps as one call
        g.forward_cached_dev_exchange(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), pos, own,
                                      mine_off, lse_off, slot * world * pay, world * pay, step + 1, stream=stream)
    if split:
        ctx.merge_parts(ctx.comm_data_ptr() + slot * world * pay * 4, world, sp.seq_parts, Hl, hd, merged.data_ptr(), stream)
        torch.cuda.synchronize(); ctx.sync()
        full = merged.cpu().numpy()
    else:
        full = np.empty(world * pay, np.float32)
        ctx.comm_read(slot * world * pay, full, stream)
        torch.cuda.synchronize(); ctx.sync()
    worst = max(worst, rel_err(full, ref))
    dist.barrier()       # a slot is rewritten two steps later; the host barrier keeps this test's reads simple
assert worst <= DECODE_TOL, worst
assert len(g.cache) == sp.local_rows(L0 + 6)
dist.barrier()
g.close(); ctx.close()
print("RANK_OK", rank, worst)
"""


@pytest.mark.parametrize("mode", ["heads", "split"])
def test_two_ranks_deliver_to_each_other(tmp_path, mode):
    """Two processes, one GPU each.  "heads": each rank owns two of the four kv-head groups.
    "split": one kv head, the ranks hold alternate positions, exchange (output, log-sum-exp)
    and merge.  Both against the unsharded oracle at the decode tolerance."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = "29541" if mode == "heads" else "29542"
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=port, WORLD_SIZE="2", NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, mode], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "RANK_OK" in o, f"rank {r}:\n{o[-3000:]}"


BATCHED_WORKER = r"""
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.path.join(sys.argv[1], "tests")); sys.path.insert(0, sys.argv[1])
import shainet_b200 as S
from helpers import Q8B, qkv, rel_err, DECODE_TOL
from oracle import oracle as O
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo")
H, KV, hd = Q8B["H"], Q8B["KV"], Q8B["hd"]
KVl, Hl = KV // world, H // world
rng = np.random.default_rng(6400)            # same stream on every rank: identical full inputs
qn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
kn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
lens = [1, 33, 700, 1500, 2900, 64]
ctx = S.AttnContext(rank)
oracles, caches = [], []
kvs = slice(rank * KVl, (rank + 1) * KVl)
for L in lens:
    kc = rng.standard_normal((KV, L, hd), dtype=np.float32)
    vc = rng.standard_normal((KV, L, hd), dtype=np.float32)
    o = O.OracleAttention(H, KV, hd, Q8B["theta"], 1e-6, q_norm=qn, k_norm=kn)
    o.import_cache(kc, vc)
    g = S.LlamaAttention(ctx, Hl, KVl, hd, Q8B["theta"], 1e-6, q_norm=qn, k_norm=kn)
    g.cache.import_(kc[kvs], vc[kvs])
    g.cache.reserve(L + 4)
    oracles.append(o); caches.append(g)
dev = torch.device("cuda", rank)
stream = torch.cuda.current_stream().cuda_stream
B = len(lens)
worst = 0.0
for step in range(3):
    q, k, v = qkv(rng, Q8B, B)
    ql = q.reshape(B, H, hd)[:, rank * Hl:(rank + 1) * Hl].reshape(B, -1).copy()
    kl = k.reshape(B, KV, hd)[:, kvs].reshape(B, -1).copy()
    vl = v.reshape(B, KV, hd)[:, kvs].reshape(B, -1).copy()
    tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (ql, kl, vl))
    out = torch.empty(B, Hl * hd, device=dev)
    S.forward_batched_dev(ctx, [g.cache for g in caches], tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(),
                          caches[0].scale, stream)
    torch.cuda.synchronize(); ctx.sync()
    mine = out.cpu()
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)              # head outputs of all ranks, before o_proj
    full = torch.stack(parts, 1).reshape(B, H * hd).numpy()
    for b, o in enumerate(oracles):
        ref = o.attend_cached(q[b:b + 1], k[b:b + 1], v[b:b + 1], threads=4)
        worst = max(worst, rel_err(full[b:b + 1], ref))
assert worst <= DECODE_TOL, worst
for b, g in enumerate(caches):
    assert g.cache_len == lens[b] + 3
    g.close()
dist.barrier()
ctx.close()
print("RANK_OK", rank, worst)
"""


def test_two_ranks_share_a_ragged_batch_by_kv_head(tmp_path):
    """Batched ragged decode with the kv heads of every sequence divided over two processes (one GPU
    each), head outputs gathered before o_proj: against one unsharded oracle per sequence."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker_batched.py"
    script.write_text(BATCHED_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29543", WORLD_SIZE="2", NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), ROOT], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o)
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "RANK_OK" in o, f"rank {r}:\n{o[-3000:]}"
