"""Writer for the reference's IBF-v1 container (32-byte preamble "INFERBIT" | u32 version | u32 header
size | u32 flags | 12 reserved, JSON header, padding to 64 bytes, tensor data), laid out as
src/ibf_loader.c:351-546 reads it and as the reference's own tests/test_ibf_loader.c writes it.
Test and benchmark infrastructure: it builds the model files that the unmodified reference
(oracle/_ref) and the GPU front load; nothing in the product path uses it."""
import json
import struct

import numpy as np

NAMES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def write_ibf(path, cfg, layers, head, emb, name="b200-parity-mini"):
    """cfg: dict(hidden, inter, n_layers, n_heads, n_kv_heads, head_dim, vocab, max_ctx, eps, theta, attn_bits, mlp_bits).
    layers[l] = ([(w, scale_bits, M, N, bits)] * 7, (input_norm_bits, post_attn_norm_bits)); head = (w, scale_bits, M, N, bits);
    emb = (int8 rows, fp16 row-scale bits, final-norm fp16 bits)."""
    embw, emb_scale, final_norm = emb
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
        wts = {nm: meta(*lins[i]) for i, nm in enumerate(NAMES)}
        wts["input_norm"] = meta(norms[0], None, cfg["hidden"], None, 16)
        wts["post_attn_norm"] = meta(norms[1], None, cfg["hidden"], None, 16)
        jl.append({"index": l, "weights": wts, "sparsity_mask": {"offset": 0, "size": 0}})
    hdr = {
        "version": 1,
        "model": {"architecture": "llama", "name": name},
        "architecture": {"num_layers": cfg["n_layers"], "hidden_size": cfg["hidden"], "num_heads": cfg["n_heads"],
                         "num_kv_heads": cfg["n_kv_heads"], "head_dim": cfg["head_dim"], "intermediate_size": cfg["inter"],
                         "vocab_size": cfg["vocab"], "max_context_length": cfg["max_ctx"], "rope_theta": cfg["theta"],
                         "norm_epsilon": cfg["eps"], "norm_type": "rmsnorm", "activation": "silu",
                         "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": False},
        "quantization": {"default_bits": cfg["mlp_bits"], "sensitive_bits": cfg["attn_bits"], "sparsity": 0.0, "block_size": 8},
        "kv_cache": {"bits": 16},
        "layers": jl,
        "embeddings": {"token_embedding": meta(embw, emb_scale, cfg["vocab"], cfg["hidden"], 8)},
        "output": {"norm": meta(final_norm, None, cfg["hidden"], None, 16), "head": meta(*head)},
    }
    hdr["data"] = {"weight_data_offset": 0, "weight_data_size": len(blob), "alignment": 64}
    js = json.dumps(hdr).encode()
    with open(path, "wb") as f:
        f.write(b"INFERBIT" + struct.pack("<III", 1, len(js), 0) + bytes(12))
        f.write(js)
        f.write(bytes((-(32 + len(js))) % 64))
        f.write(bytes(blob))
