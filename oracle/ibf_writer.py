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


def write_ibf_v5(path, tensors, raw_tensors=None, config=None, reserve_pad=64):
    """Writes a product-quantised model file as the reference's readers take it (src/pq_decode.c:391-546, :726-852): 32-byte
    preamble ("INFERBIT", version 5, header length), JSON header padded with spaces, then the blocks.
    tensors: {name: dict(format=..., M, N, G, K, n_levels, K_l2=0, rotate=False, l2_packed_bits=0, n_outlier=0, blocks={key: ndarray})};
    raw_tensors: {name: ndarray}; config: any JSON-able dict."""
    dtype_names = {"float32": "float32", "float16": "float16", "int32": "int32", "int16": "int16", "int8": "int8", "uint8": "uint8", "uint16": "uint16"}
    blobs, off = [], 0

    def place(arr):
        nonlocal off
        b = np.ascontiguousarray(arr).tobytes()
        at = off
        blobs.append(b)
        off += len(b)
        pad = (-off) % 16
        if pad:
            blobs.append(bytes(pad)); off += pad
        return {"offset": at, "size": len(b)}

    header = {"tensors": {}}
    for name, t in tensors.items():
        tm = {"format": t["format"], "shape": [t["M"], t["N"]], "G": t["G"], "K": t["K"], "n_levels": t["n_levels"],
              "rotate": bool(t.get("rotate", False)), "K_l2": t.get("K_l2", 0)}
        if t.get("l2_packed_bits", 0):
            tm["l2_packed_bits"] = t["l2_packed_bits"]
        if t.get("n_outlier", 0):
            tm["outlier"] = {"n_cols": t["n_outlier"]}
        for key, arr in t["blocks"].items():
            tm[key] = place(arr)
        header["tensors"][name] = tm
    if raw_tensors:
        header["raw_tensors"] = {}
        for name, arr in raw_tensors.items():
            arr = np.ascontiguousarray(arr)
            blk = place(arr)
            header["raw_tensors"][name] = {"dtype": dtype_names[str(arr.dtype)], "shape": list(arr.shape), **blk}
    if config is not None:
        header["config"] = config
    # the header names its own length through weight_data_start: reserve first, then fill in
    header["weight_data_start"] = 0
    reserve = len(json.dumps(header).encode()) + reserve_pad
    header["weight_data_start"] = 32 + reserve
    text = json.dumps(header).encode()
    assert len(text) <= reserve
    with open(path, "wb") as f:
        f.write(b"INFERBIT" + struct.pack("<II", 5, reserve) + bytes(16))
        f.write(text + b" " * (reserve - len(text)))
        for b in blobs:
            f.write(b)
    return header
