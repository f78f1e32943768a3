"""shainet_attn_decode_noalloc: the decode entry for hosts that cannot let the
library allocate device memory (a server whose own pool owns the whole GPU
budget; a token loop that must not hit cudaMalloc's device-wide sync).  Its
split partials sit in a fixed array inside the library, so the test calls it
twice in a row - the second call reuses what the first left there - and checks
each result against the library's existing attention_kv_f32 entry on the same
buffers AND against the CPU oracle's attention over the same cache
(attention_heads_cpu, llama_block.cr:302-401), both within the decode tolerance
max|y-ref|/max|ref| <= 1e-5.
Collected last on purpose: a failure here cannot hide the other tests."""
import numpy as np
import pytest

from helpers import DECODE_TOL, Q30, L1B, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,ctx_len", [(Q30, 6000), (L1B, 4096)], ids=["qwen3_30b_6k", "llama1b_4k"])
def test_noalloc_decode_matches_existing_entry_and_oracle_twice(shape, ctx_len):
    import torch
    from oracle import oracle as O
    from shainet_b200 import _lib, build
    build.build()
    lib = _lib.load()
    H, KV, hd = shape["H"], shape["KV"], shape["hd"]
    cap = ctx_len + 8
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev); g.manual_seed(1234)
    kc = torch.randn(KV, cap, hd, device=dev, generator=g)
    vc = torch.randn(KV, cap, hd, device=dev, generator=g)
    o = O.OracleAttention(H, KV, hd, shape["theta"], 1e-6)
    o.import_cache(kc[:, :ctx_len + 1].cpu().numpy(), vc[:, :ctx_len + 1].cpu().numpy())
    scale = float(np.float32(1.0 / np.sqrt(float(hd))))
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                       # two calls in a row share the fixed scratch
        start = ctx_len - 1 + call              # visible rows 0..start; the second call sees one more row
        q_raw = torch.randn(H * hd, generator=torch.Generator().manual_seed(77 + call))
        # The entry takes q already rotated, the oracle's attend_only rotates q itself
        # (llama_block.cr:332-344): the library is handed the same rotation, computed here in
        # fp32 with the block's formula (angle = f32(pos) * inv_freq, half-split pairs).
        inv = o.inv_freq()
        ang = (np.float32(start) * inv).astype(np.float32)
        c, s_ = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
        x = q_raw.numpy().reshape(H, hd)
        x0, x1 = x[:, :hd // 2], x[:, hd // 2:]
        q_rot = np.concatenate([x0 * c - x1 * s_, x1 * c + x0 * s_], axis=1).astype(np.float32).reshape(-1)
        q = torch.from_numpy(q_rot).to(dev)
        oracle_out = o.attend_only(q_raw.numpy().reshape(1, -1), start, threads=4)[0]
        ref = torch.zeros(H * hd, device=dev)
        ws = torch.zeros(H * (start + 1), device=dev)
        got = torch.full((H * hd,), float("nan"), device=dev)
        torch.cuda.synchronize()
        lib.attention_kv_f32(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ref.data_ptr(), ws.data_ptr(), 1, start, H,
                             H // KV, hd, cap, scale)
        rc = lib.shainet_attn_decode_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), got.data_ptr(), start, H,
                                             H // KV, hd, cap, scale, stream)
        assert rc == 0, lib.shainet_attn_last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        assert rel_err(got.cpu().numpy(), ref.cpu().numpy()) <= DECODE_TOL, call
        assert rel_err(got.cpu().numpy(), oracle_out) <= DECODE_TOL, (call, rel_err(got.cpu().numpy(), oracle_out))


def test_noalloc_rejects_what_does_not_fit():
    import torch
    from shainet_b200 import _lib, build
    build.build()
    lib = _lib.load()
    dev = torch.device("cuda:0")
    buf = torch.zeros(4096, device=dev)
    p = buf.data_ptr()
    # head_dim 8 has no split-K instance
    assert lib.shainet_attn_decode_noalloc(p, p, p, p, 3, 8, 2, 8, 16, 0.35, None) == _lib.E_UNSUPPORTED
    assert b"head_dim" in lib.shainet_attn_last_error()
    # 16384 query heads would need far more than the fixed 4 MiB of partials
    assert lib.shainet_attn_decode_noalloc(p, p, p, p, 100000, 16384, 16, 128, 100001, 0.088, None) == _lib.E_UNSUPPORTED
    assert b"exceeds the fixed scratch" in lib.shainet_attn_last_error()
    assert lib.shainet_attn_decode_noalloc(None, p, p, p, 3, 8, 2, 64, 16, 0.125, None) == _lib.E_INVALID
    assert lib.shainet_attn_decode_noalloc(p, p, p, p, 16, 8, 2, 64, 16, 0.125, None) == _lib.E_INVALID   # start_pos >= capacity
