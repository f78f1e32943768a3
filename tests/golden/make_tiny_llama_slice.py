"""Cut the part of the reference's tiny-llama fixture that its cache-consistency
spec touches (spec/rope_kv_cache_spec.cr:30-59) into a small .npz.

The fixture (spec/test_data/tiny-llama/model.safetensors, 4.1 MB, HF
tiny-random LLaMA: hidden 16, 4 heads, 4 KV heads, 2 layers, FFN 64, eps 1e-6,
theta 1e4) is dominated by a 32000 x 16 embedding table of which the spec reads
four rows (tokens 1, 42, 100, 7).  This script keeps those rows and the two
layers' weights, transposed from HF [out, in] to the reference's [in, out]
(src/shainet/hf_loader.cr:326-329).  It only runs where the reference tree is
mounted; the tests read the .npz.

Run:  python tests/golden/make_tiny_llama_slice.py [reference_root]
"""
import json
import os
import struct
import sys

import numpy as np

TOKENS = [1, 42, 100, 7]


def read_safetensors(path):
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        assert meta["dtype"] == "F32", (name, meta["dtype"])
        a, b = meta["data_offsets"]
        out[name] = np.frombuffer(blob[a:b], dtype="<f4").reshape(meta["shape"]).copy()
    return out


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SHAINET_REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: make_tiny_llama_slice.py <path of a SHAInet checkout> (or set SHAINET_REFERENCE_ROOT)")
    d = os.path.join(root, "spec", "test_data", "tiny-llama")
    cfg = json.load(open(os.path.join(d, "config.json")))
    t = read_safetensors(os.path.join(d, "model.safetensors"))
    out = {
        "tokens": np.array(TOKENS, np.int32),
        "embed_rows": t["model.embed_tokens.weight"][TOKENS],
        "hidden_size": np.int32(cfg["hidden_size"]),
        "num_heads": np.int32(cfg["num_attention_heads"]),
        "num_kv_heads": np.int32(cfg["num_key_value_heads"]),
        "num_layers": np.int32(cfg["num_hidden_layers"]),
        "eps": np.float64(cfg["rms_norm_eps"]),
        "rope_theta": np.float64(cfg["rope_theta"]),
    }
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        for short, name in [("w_q", "self_attn.q_proj"), ("w_k", "self_attn.k_proj"), ("w_v", "self_attn.v_proj"),
                            ("w_o", "self_attn.o_proj"), ("gate", "mlp.gate_proj"), ("up", "mlp.up_proj"),
                            ("down", "mlp.down_proj")]:
            out[f"l{l}.{short}"] = np.ascontiguousarray(t[p + name + ".weight"].T)
        out[f"l{l}.norm1"] = t[p + "input_layernorm.weight"]
        out[f"l{l}.norm2"] = t[p + "post_attention_layernorm.weight"]
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_llama_slice.npz")
    np.savez_compressed(dst, **out)
    print(dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
