"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no model file or dataset exists for them).

Packed weights are returned as ``uint8`` numpy arrays ``[rows, row_bytes]`` in
the GGUF block layouts (src/runtime/quants.h:23-26 of the reference). Value
distributions:

  Q4_K  f16 d ~ U[0.001, 0.02], f16 dmin ~ U[0, 0.01]; the 12 scale bytes and
        128 quant bytes are uniform random bytes, which makes every 6-bit
        scale / min uniform on 0..63 and every 4-bit quant uniform on 0..15
        (the packing is a bijection between 12 bytes and 16 six-bit fields)
  Q6_K  f16 d ~ U[0.001, 0.02]; int8 sub-block scales ~ U{-63..63}; ql / qh
        uniform random bytes (6-bit quants uniform on 0..63)
  Q8_0  f16 d ~ U[0.001, 0.02]; int8 quants ~ U{-127..127}

Every tensor draws from its own ``numpy.random.Generator(PCG64(seed))`` whose
seed is derived from (global seed, tensor name), so tensors can be generated in
any order or one at a time.
"""
import zlib

import numpy as np

from . import capi

LLAMA3_8B = dict(n_layer=32, n_embd=4096, n_head=32, n_kv_head=8, head_dim=128, n_ff=14336,
                 n_vocab=128256, max_kv=8192 + 256, rope_base=500000.0, eps=1e-5)

# Q4_K_M recipe of the benchmark: Q6_K for attn_v, ffn_down and the output head.
Q4_K_M = {"wq": capi.Q4_K, "wk": capi.Q4_K, "wv": capi.Q6_K, "wo": capi.Q4_K, "gate": capi.Q4_K,
          "up": capi.Q4_K, "down": capi.Q6_K, "output": capi.Q6_K, "tok_embd": capi.Q6_K}
LAYER_TENSORS = ["wq", "wk", "wv", "wo", "gate", "up", "down"]


def rng_for(seed, name):
    return np.random.Generator(np.random.PCG64([seed, zlib.crc32(name.encode())]))


def _f16_uniform(rng, lo, hi, n):
    return rng.uniform(lo, hi, n).astype(np.float32).astype(np.float16).view(np.uint16)


def q4k_tensor(rng, rows, cols):
    nb = rows * (cols // 256)
    blk = np.empty((nb, 144), dtype=np.uint8)
    hdr = blk[:, :4].view(np.uint16)
    hdr[:, 0] = _f16_uniform(rng, 0.001, 0.02, nb)
    hdr[:, 1] = _f16_uniform(rng, 0.0, 0.01, nb)
    blk[:, 4:] = rng.integers(0, 256, (nb, 140), dtype=np.uint8)
    return blk.reshape(rows, -1)


def q6k_tensor(rng, rows, cols):
    nb = rows * (cols // 256)
    blk = np.empty((nb, 210), dtype=np.uint8)
    blk[:, :192] = rng.integers(0, 256, (nb, 192), dtype=np.uint8)
    blk[:, 192:208] = rng.integers(-63, 64, (nb, 16), dtype=np.int8).view(np.uint8)
    blk[:, 208:210] = _f16_uniform(rng, 0.001, 0.02, nb).reshape(nb, 1).view(np.uint8)
    return blk.reshape(rows, -1)


def q8_0_tensor(rng, rows, cols):
    nb = rows * (cols // 32)
    blk = np.empty((nb, 34), dtype=np.uint8)
    blk[:, :2] = _f16_uniform(rng, 0.001, 0.02, nb).reshape(nb, 1).view(np.uint8)
    blk[:, 2:] = rng.integers(-127, 128, (nb, 32), dtype=np.int8).view(np.uint8)
    return blk.reshape(rows, -1)


def q5_0_tensor(rng, rows, cols):
    nb = rows * (cols // 32)
    blk = np.empty((nb, 22), dtype=np.uint8)
    blk[:, :2] = _f16_uniform(rng, 0.001, 0.02, nb).reshape(nb, 1).view(np.uint8)
    blk[:, 2:] = rng.integers(0, 256, (nb, 20), dtype=np.uint8)
    return blk.reshape(rows, -1)


def quant_tensor(fmt, rng, rows, cols):
    if fmt == capi.Q4_K:
        return q4k_tensor(rng, rows, cols)
    if fmt == capi.Q6_K:
        return q6k_tensor(rng, rows, cols)
    if fmt == capi.Q8_0:
        return q8_0_tensor(rng, rows, cols)
    if fmt == capi.Q5_0:
        return q5_0_tensor(rng, rows, cols)
    if fmt == capi.F32:
        return rng.standard_normal((rows, cols), dtype=np.float32).view(np.uint8).reshape(rows, -1)
    raise ValueError(fmt)


def config0(seed=0):
    """Configuration 0 of the benchmark: one decode attention (32/8 heads, d 128,
    KV 1024, f16 cache ~ N(0,1)/sqrt(128), f32 q ~ N(0,1)) and one 4096x4096 Q4_K
    matvec with an f32 N(0,1) activation. K/V are laid out [n_kv_head][kv][d]."""
    rng = np.random.Generator(np.random.PCG64(seed))
    q = rng.standard_normal((32, 128), dtype=np.float32)
    k = (rng.standard_normal((8, 1024, 128), dtype=np.float32) / np.sqrt(np.float32(128))).astype(np.float16)
    v = (rng.standard_normal((8, 1024, 128), dtype=np.float32) / np.sqrt(np.float32(128))).astype(np.float16)
    w = q4k_tensor(rng, 4096, 4096)
    x = rng.standard_normal(4096, dtype=np.float32)
    return dict(q=q, k=k, v=v, w=w, x=x, scale=float(1.0 / np.sqrt(np.float32(128))))


def layer_shapes(cfg):
    E, QD, KD, F = cfg["n_embd"], cfg["n_head"] * cfg["head_dim"], cfg["n_kv_head"] * cfg["head_dim"], cfg["n_ff"]
    return {"wq": (QD, E), "wk": (KD, E), "wv": (KD, E), "wo": (E, QD), "gate": (F, E), "up": (F, E),
            "down": (E, F)}


def llama_tensor(cfg, seed, name, layer=None, recipe=Q4_K_M):
    """One packed weight tensor of the synthetic model, by name."""
    if name in ("output", "tok_embd"):
        rows, cols = cfg["n_vocab"], cfg["n_embd"]
        tag = name
    else:
        rows, cols = layer_shapes(cfg)[name]
        tag = "L%d.%s" % (layer, name)
    return quant_tensor(recipe[name], rng_for(seed, tag), rows, cols)


def llama_norm(cfg, seed, name, layer=None):
    """f32 norm weights ~ U[0.9, 1.1]."""
    tag = name if layer is None else "L%d.%s" % (layer, name)
    return rng_for(seed, tag).uniform(0.9, 1.1, cfg["n_embd"]).astype(np.float32)


def llama_kv(cfg, seed, layer, n_pos, std=0.1):
    """Prefilled f16 K and V of one layer, [n_kv_head][n_pos][head_dim] ~ N(0, std)."""
    rng = rng_for(seed, "L%d.kv" % layer)
    shape = (cfg["n_kv_head"], n_pos, cfg["head_dim"])
    k = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float16)
    v = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float16)
    return k, v


def model_weight_bytes(cfg, recipe=Q4_K_M):
    """Packed weight bytes + f32 norm bytes one decode step reads (embedding row excluded)."""
    total = 0
    for name, (rows, cols) in layer_shapes(cfg).items():
        total += rows * capi.row_bytes(recipe[name], cols)
    total = cfg["n_layer"] * (total + 2 * cfg["n_embd"] * 4)
    total += cfg["n_vocab"] * capi.row_bytes(recipe["output"], cfg["n_embd"]) + cfg["n_embd"] * 4
    return total


# ---- device-side generators (benchmark set-up) --------------------------------
# Same layouts and value distributions as above, drawn with torch on the GPU so
# that the 4.9 GB model of the benchmark is ready in about a second instead of
# half a minute of host generation + upload. (Different random stream than the
# numpy generators: use those whenever a host-side checker must see the same bytes.)

def device_quant_tensor(fmt, rows, cols, gen):
    import torch
    nb = rows * (cols // capi.BLK_ELEMS[fmt])
    bb = capi.BLK_BYTES[fmt]
    dev = gen.device
    w = torch.randint(0, 256, (nb, bb), dtype=torch.uint8, device=dev, generator=gen)

    def f16_uniform(lo, hi):
        return (torch.rand(nb, device=dev, generator=gen) * (hi - lo) + lo).half().view(torch.uint8).reshape(nb, 2)

    if fmt == capi.Q4_K:
        w[:, 0:2] = f16_uniform(0.001, 0.02)
        w[:, 2:4] = f16_uniform(0.0, 0.01)
    elif fmt == capi.Q6_K:
        w[:, 192:208] = torch.randint(-63, 64, (nb, 16), dtype=torch.int8, device=dev, generator=gen).view(torch.uint8)
        w[:, 208:210] = f16_uniform(0.001, 0.02)
    elif fmt == capi.Q8_0:
        w[:, 0:2] = f16_uniform(0.001, 0.02)
    else:
        raise ValueError(fmt)
    return w.reshape(rows, -1)


def device_llama(dec, cfg, seed, n_prefill, kv_std=0.1, recipe=Q4_K_M, skip_ffn=()):
    """Fills a fast_llm_b200.decoder.Decoder with a synthetic model generated on
    its device and prefills n_prefill KV positions ~ N(0, kv_std). A
    tensor-parallel decoder gets tensors of its share's shapes (drawn directly,
    not sliced from a whole model: the values are synthetic either way). Layers in
    skip_ffn get no gate / up / down (the caller sets a mixture-of-experts block there).
    Returns the list of tensors kept alive."""
    import ctypes as C
    import torch
    from . import tp
    dev = torch.device("cuda", dec.ctx.device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed * 64 + dec.rank)   # this rank's slices
    rep = torch.Generator(device=dev)
    rep.manual_seed(seed * 64 + 63)         # tensors every rank holds whole: norms, embedding table
    keep = []
    shapes = layer_shapes(dec.loc)
    for l in range(cfg["n_layer"]):
        for i, name in enumerate(LAYER_TENSORS):
            if l in skip_ffn and name in ("gate", "up", "down"):
                continue
            rows, cols = shapes[name]
            w = device_quant_tensor(recipe[name], rows, cols, gen)
            if name in tp.COL_SPLIT and w.shape[1] % 16:
                w = torch.nn.functional.pad(w, (0, 16 - w.shape[1] % 16)).contiguous()
            dec.set_layer_tensor(l, i, recipe[name], w)
        an = torch.rand(cfg["n_embd"], device=dev, generator=rep) * 0.2 + 0.9
        fn = torch.rand(cfg["n_embd"], device=dev, generator=rep) * 0.2 + 0.9
        dec.set_layer_norms(l, an, fn)
        if n_prefill:
            kp, vp = dec.kv_ptrs(l)
            for ptr in (kp, vp):
                nkv = dec.loc["n_kv_head"]
                t = (torch.randn((nkv, n_prefill, cfg["head_dim"]), device=dev, generator=gen) * kv_std).half()
                full = torch.zeros((nkv, cfg["max_kv"], cfg["head_dim"]), dtype=torch.float16, device=dev)
                full[:, :n_prefill] = t
                torch.cuda.synchronize(dev)
                # copy into the decoder's cache (the source may be a device pointer)
                capi._ck(dec.lib.fl_b200_upload(dec.ctx._h, C.c_void_p(ptr), C.c_void_p(full.data_ptr()),
                                                C.c_size_t(full.numel() * 2)))
    for which, name in ((capi.G_TOK_EMBD, "tok_embd"), (capi.G_OUTPUT, "output")):
        rows = cfg["n_vocab"] if name == "tok_embd" else dec.loc["n_vocab"]   # the embedding table is whole on every rank
        w = device_quant_tensor(recipe[name], rows, cfg["n_embd"], rep if name == "tok_embd" else gen)
        dec.set_global(which, recipe[name], w)
    on = torch.rand(cfg["n_embd"], device=dev, generator=rep) * 0.2 + 0.9
    dec.set_out_norm(on)
    torch.cuda.synchronize(dev)
    return keep


def device_seqs(dec, cfg, n_seq, n_prefill, seed=7, kv_std=0.1):
    """Sets a decoder up for n_seq independent sequences (Decoder.seqs_init) and prefills n_prefill positions of every
    sequence's cache with f16 ~ N(0, kv_std), generated on the device."""
    import ctypes as C
    import torch
    dev = torch.device("cuda", dec.ctx.device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    dec.seqs_init(n_seq)
    nkv = dec.loc["n_kv_head"]
    for l in range(cfg["n_layer"]):
        for s in range(n_seq):
            for ptr in dec.seqs_kv_ptrs(l, s):
                t = (torch.randn((nkv, n_prefill, cfg["head_dim"]), device=dev, generator=gen) * kv_std).half()
                full = torch.zeros((nkv, cfg["max_kv"], cfg["head_dim"]), dtype=torch.float16, device=dev)
                full[:, :n_prefill] = t
                torch.cuda.synchronize(dev)
                capi._ck(dec.lib.fl_b200_upload(dec.ctx._h, C.c_void_p(ptr), C.c_void_p(full.data_ptr()), C.c_size_t(full.numel() * 2)))
    for s in range(n_seq):
        dec.seqs_set_pos(s, n_prefill)
