"""Host-side logic of the multi-GPU partition: the shard plan, and - with two
gloo ranks on CPU - that head-sharded and sequence-split attention, gathered and
merged the way the GPU path does it, reproduce the unsharded CPU oracle."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plan_head_groups_then_sequence_parts():
    from shainet_b200.sharding import plan
    p = plan(4, 2, 32, 4)
    assert (p.groups, p.seq_parts, p.kv_begin, p.kv_count, p.head_begin, p.head_count) == (4, 1, 2, 1, 16, 8)
    p = plan(2, 1, 32, 8)
    assert (p.kv_begin, p.kv_count, p.head_begin, p.head_count) == (4, 4, 16, 16)
    p = plan(8, 5, 32, 4)         # more ranks than kv heads: 4 groups x 2 sequence parts
    assert (p.groups, p.seq_parts, p.group, p.seq_part, p.kv_begin, p.head_begin, p.head_count) == (4, 2, 2, 1, 2, 16, 8)
    assert p.owns_position(7) and not p.owns_position(8)
    assert [plan(8, r, 32, 4).local_rows(32769) for r in (0, 1)] == [16385, 16384]
    with pytest.raises(ValueError):
        plan(3, 0, 32, 4)
    with pytest.raises(ValueError):
        plan(6, 0, 32, 4)


def test_merge_parts_host_matches_unsplit_softmax():
    from shainet_b200.sharding import merge_parts_host
    rng = np.random.default_rng(0)
    H, hd, L = 3, 8, 50
    s = rng.standard_normal((H, L)); v = rng.standard_normal((L, hd))
    full = np.stack([np.exp(s[h] - s[h].max()) @ v / np.exp(s[h] - s[h].max()).sum() for h in range(H)])
    outs, lses = [], []
    for part in range(2):
        idx = np.arange(part, L, 2)
        e = np.exp(s[:, idx] - s[:, idx].max(axis=1, keepdims=True))
        outs.append(e @ v[idx] / e.sum(axis=1, keepdims=True))
        lses.append(s[:, idx].max(axis=1) + np.log(e.sum(axis=1)))
    assert np.allclose(merge_parts_host(np.stack(outs), np.stack(lses)), full, atol=1e-6)
    # a part that holds no row contributes nothing
    outs.append(np.zeros((H, hd))); lses.append(np.full(H, -np.inf))
    assert np.allclose(merge_parts_host(np.stack(outs), np.stack(lses)), full, atol=1e-6)


WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
    import numpy as np, torch, torch.distributed as dist
    from oracle import oracle as O
    from shainet_b200.sharding import plan, merge_parts_host
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    H, hd, T0, steps = 8, 16, 21, 3
    for KV in (4, 1):                       # KV=4: head groups; KV=1 with 2 ranks: sequence split
        p = plan(world, rank, H, KV)
        rng = np.random.default_rng(99)     # same stream on every rank
        full = O.OracleAttention(H, KV, hd, 10000.0)
        mine = O.OracleAttention(p.head_count, p.kv_count, hd, 10000.0)
        qs = rng.standard_normal((T0 + steps, H * hd)).astype(np.float32)
        ks = rng.standard_normal((T0 + steps, KV * hd)).astype(np.float32)
        vs = rng.standard_normal((T0 + steps, KV * hd)).astype(np.float32)
        full.attend_cached(qs[:T0], ks[:T0], vs[:T0])
        kc, vc = full.export_cache()        # rotated rows of the prefill
        rows = np.arange(p.seq_part, T0, p.seq_parts)
        mine.import_cache(kc[p.kv_begin:p.kv_begin + p.kv_count][:, rows], vc[p.kv_begin:p.kv_begin + p.kv_count][:, rows])
        hs = slice(p.head_begin * hd, (p.head_begin + p.head_count) * hd)
        kvs = slice(p.kv_begin * hd, (p.kv_begin + p.kv_count) * hd)
        for t in range(T0, T0 + steps):
            ref = full.attend_cached(qs[t:t + 1], ks[t:t + 1], vs[t:t + 1])[0]
            if p.owns_position(t):          # this rank stores the new row: rotate it with the full oracle's arithmetic
                kc, vc = full.export_cache()
                rows = np.append(rows, t)
                mine.import_cache(kc[p.kv_begin:p.kv_begin + p.kv_count][:, rows], vc[p.kv_begin:p.kv_begin + p.kv_count][:, rows])
            # scores/softmax over this rank's rows only, with the query rotated at position t
            kk, vv = mine.export_cache()
            qrot = O.OracleAttention(p.head_count, p.head_count, hd, 10000.0)
            dummy = np.zeros((t, p.head_count * hd), np.float32)
            q1 = qs[t:t + 1, hs]
            # rotate q at position t: append t dummy rows first so that the next row sits at position t
            qrot.import_cache(np.zeros((p.head_count, t, hd), np.float32), np.zeros((p.head_count, t, hd), np.float32))
            qrot.attend_cached(q1, q1, q1)
            qr = qrot.export_cache()[0][:, t, :]            # [heads, hd], q rotated at position t
            g = p.head_count // p.kv_count
            out = np.zeros((p.head_count, hd)); lse = np.zeros(p.head_count)
            for h in range(p.head_count):
                sc = (kk[h // g] @ qr[h]) * np.float32(1.0 / np.sqrt(hd))
                e = np.exp(sc - sc.max())
                out[h] = e @ vv[h // g] / e.sum()
                lse[h] = sc.max() + np.log(e.sum())
            payload = torch.from_numpy(np.concatenate([out.ravel(), lse]).astype(np.float32))
            gathered = [torch.empty_like(payload) for _ in range(world)]
            dist.all_gather(gathered, payload)
            gathered = np.stack([x.numpy() for x in gathered])      # [world, Hr*hd + Hr]
            Hr = p.head_count
            merged = []
            for grp in range(p.groups):
                part = gathered[grp * p.seq_parts:(grp + 1) * p.seq_parts]
                merged.append(merge_parts_host(part[:, :Hr * hd].reshape(p.seq_parts, Hr, hd), part[:, Hr * hd:]))
            got = np.concatenate(merged).ravel()
            err = np.abs(got - ref).max() / np.abs(ref).max()
            assert err < 2e-6, (KV, t, err)
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_two_gloo_ranks_reproduce_the_unsharded_oracle(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)],
                       capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("ok") == 2


BATCHED_WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
    import numpy as np, torch, torch.distributed as dist
    from oracle import oracle as O
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    H, KV, hd = 8, 4, 16
    Hl, KVl = H // world, KV // world
    rng = np.random.default_rng(123)        # same stream on every rank
    lens = [1, 9, 40, 17]
    B = len(lens)
    full, mine = [], []
    kvs = slice(rank * KVl, (rank + 1) * KVl)
    for L in lens:
        kc = rng.standard_normal((KV, L, hd)).astype(np.float32)
        vc = rng.standard_normal((KV, L, hd)).astype(np.float32)
        f = O.OracleAttention(H, KV, hd, 10000.0); f.import_cache(kc, vc); full.append(f)
        m = O.OracleAttention(Hl, KVl, hd, 10000.0); m.import_cache(kc[kvs], vc[kvs]); mine.append(m)
    for step in range(3):
        q = rng.standard_normal((B, H * hd)).astype(np.float32)
        k = rng.standard_normal((B, KV * hd)).astype(np.float32)
        v = rng.standard_normal((B, KV * hd)).astype(np.float32)
        # this rank's columns of the lock-step rows: its query heads and its kv heads
        ql = q.reshape(B, H, hd)[:, rank * Hl:(rank + 1) * Hl].reshape(B, -1)
        kl = k.reshape(B, KV, hd)[:, kvs].reshape(B, -1)
        vl = v.reshape(B, KV, hd)[:, kvs].reshape(B, -1)
        out = np.stack([mine[b].attend_cached(ql[b:b + 1], kl[b:b + 1], vl[b:b + 1])[0] for b in range(B)])
        payload = torch.from_numpy(out.astype(np.float32))               # [B, Hl*hd]
        gathered = torch.empty(world, B, Hl * hd)
        dist.all_gather_into_tensor(gathered.view(-1), payload.view(-1))  # the layout the bench gathers into
        got = gathered.permute(1, 0, 2).reshape(B, H * hd).numpy()        # [B, rank-major head blocks] = [B, H*hd]
        for b in range(B):
            ref = full[b].attend_cached(q[b:b + 1], k[b:b + 1], v[b:b + 1])[0]
            assert np.array_equal(got[b], ref), (step, b)                  # the same arithmetic per head: exact
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_two_gloo_ranks_share_a_ragged_batch_by_kv_head(tmp_path):
    """Batched decode with the kv heads of every sequence divided over the ranks: the per-rank column
    slices and the [rank][sequence][local heads] gather layout reassemble the unsharded rows exactly."""
    script = tmp_path / "worker_batched.py"
    script.write_text(BATCHED_WORKER.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29544", str(script)],
                       capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("ok") == 2
