"""A small llama-shaped model as seeded tensors, written as an IBF-v1 file by oracle/ibf_writer.py.
Used by make_golden.py to run the unmodified reference's inferbit_load / inferbit_forward, and by the
tests to rebuild the identical tensors from the seed."""

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
        # o_proj may be stored at its own width: the converter writes it at the default width while q, k, v
        # take the sensitive one (src/convert.c:572-578)
        lins = [lin(M, N, cfg["attn_bits"] if i <= 2 else (cfg.get("o_bits", cfg["attn_bits"]) if i == 3 else cfg["mlp_bits"]))
                for i, (M, N) in enumerate(shapes)]
        norms = (fp16_bits(rng.uniform(0.9, 1.1, H)), fp16_bits(rng.uniform(0.9, 1.1, H)))
        layers.append((lins, norms))
    head = lin(V, H, cfg["head_bits"])
    emb = (rng.integers(-127, 128, (V, H), dtype=np.int8), fp16_bits(rng.uniform(0.005, 0.02, V)), fp16_bits(rng.uniform(0.9, 1.1, H)))
    return layers, head, emb


def write_ibf(path, cfg=CFG, seed=SEED):
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    from oracle import ibf_writer
    layers, head, emb = tensors(seed, cfg)
    ibf_writer.write_ibf(path, cfg, layers, head, emb)
