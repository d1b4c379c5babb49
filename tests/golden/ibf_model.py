"""A small llama-shaped model as seeded tensors, and a writer for the reference's IBF-v1 container
(32-byte preamble "INFERBIT" | u32 version | u32 header size | u32 flags | 12 reserved, JSON header,
padding to 64 bytes, tensor data; layout as read by src/ibf_loader.c:351-546 and as the reference's own
tests/test_ibf_loader.c writes it). Used by make_golden.py to run the unmodified reference's
inferbit_load / inferbit_forward, and by the tests to rebuild the identical tensors from the seed."""
import json
import struct

import numpy as np

CFG = dict(hidden=256, inter=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64, vocab=384, max_ctx=64,
           eps=1e-5, theta=10000.0, attn_bits=8, mlp_bits=4, head_bits=8)
SEED = 777
NAMES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def fp16_bits(x):
    return np.asarray(x, np.float32).astype(np.float16).view(np.uint16)


def tensors(seed=SEED, cfg=CFG):
    """-> (layers, head, embedding): layers[l] = ([(w, scale_bits, M, N, bits)] * 7, (in_norm, post_norm))"""
    rng = np.random.default_rng(seed)
    H, I, kv, V = cfg["hidden"], cfg["inter"], cfg["n_kv_heads"] * cfg["head_dim"], cfg["vocab"]
    shapes = [(H, H), (kv, H), (kv, H), (H, H), (I, H), (I, H), (H, I)]

    def lin(M, N, bits):
        if bits == 8:
            w = rng.integers(-127, 128, (M, N), dtype=np.int8)
            s = fp16_bits(rng.uniform(0.2, 1.0, M) / (np.sqrt(N) * 73.0))
        else:
            w = rng.integers(0, 256, (M, N // 2), dtype=np.uint8)
            s = fp16_bits(rng.uniform(0.2, 1.0, M) / (np.sqrt(N) * 4.6))
        return w, s, M, N, bits
    layers = []
    for _ in range(cfg["n_layers"]):
        lins = [lin(M, N, cfg["attn_bits"] if i <= 3 else cfg["mlp_bits"]) for i, (M, N) in enumerate(shapes)]
        norms = (fp16_bits(rng.uniform(0.9, 1.1, H)), fp16_bits(rng.uniform(0.9, 1.1, H)))
        layers.append((lins, norms))
    head = lin(V, H, cfg["head_bits"])
    emb = (rng.integers(-127, 128, (V, H), dtype=np.int8), fp16_bits(rng.uniform(0.005, 0.02, V)), fp16_bits(rng.uniform(0.9, 1.1, H)))
    return layers, head, emb


def write_ibf(path, cfg=CFG, seed=SEED):
    layers, head, (emb, emb_scale, final_norm) = tensors(seed, cfg)
    blob = bytearray()

    def put(arr):
        while len(blob) % 64:
            blob.append(0)
        off = len(blob)
        blob.extend(np.ascontiguousarray(arr).tobytes())
        return off, arr.nbytes

    def meta(w, s, M, N, bits):
        off, size = put(w)
        if s is None:
            return {"offset": off, "size": size, "shape": [M] if N is None else [N, M], "bits": bits, "scale_offset": 0, "scale_size": 0, "has_bias": False}
        soff, ssize = put(s)
        return {"offset": off, "size": size, "shape": [N, M], "bits": bits, "scale_offset": soff, "scale_size": ssize, "has_bias": False}
    jl = []
    for l, (lins, norms) in enumerate(layers):
        wts = {name: meta(*lins[i]) for i, name in enumerate(NAMES)}
        wts["input_norm"] = meta(norms[0], None, cfg["hidden"], None, 16)
        wts["post_attn_norm"] = meta(norms[1], None, cfg["hidden"], None, 16)
        jl.append({"index": l, "weights": wts, "sparsity_mask": {"offset": 0, "size": 0}})
    hdr = {
        "version": 1,
        "model": {"architecture": "llama", "name": "b200-parity-mini"},
        "architecture": {"num_layers": cfg["n_layers"], "hidden_size": cfg["hidden"], "num_heads": cfg["n_heads"],
                         "num_kv_heads": cfg["n_kv_heads"], "head_dim": cfg["head_dim"], "intermediate_size": cfg["inter"],
                         "vocab_size": cfg["vocab"], "max_context_length": cfg["max_ctx"], "rope_theta": cfg["theta"],
                         "norm_epsilon": cfg["eps"], "norm_type": "rmsnorm", "activation": "silu",
                         "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": False},
        "quantization": {"default_bits": cfg["mlp_bits"], "sensitive_bits": cfg["attn_bits"], "sparsity": 0.0, "block_size": 8},
        "kv_cache": {"bits": 16},
        "layers": jl,
        "embeddings": {"token_embedding": meta(emb, emb_scale, cfg["vocab"], cfg["hidden"], 8)},
        "output": {"norm": meta(final_norm, None, cfg["hidden"], None, 16), "head": meta(*head)},
    }
    hdr["data"] = {"weight_data_offset": 0, "weight_data_size": len(blob), "alignment": 64}
    js = json.dumps(hdr).encode()
    with open(path, "wb") as f:
        f.write(b"INFERBIT" + struct.pack("<III", 1, len(js), 0) + bytes(12))
        f.write(js)
        f.write(bytes((-(32 + len(js))) % 64))
        f.write(bytes(blob))
