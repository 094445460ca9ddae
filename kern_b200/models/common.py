"""Shared pieces of the manifest generators: the built-in kernel module index, op builders for the
hand-written kernels (their launch ABI in one place), and a safetensors writer for synthetic
random-init checkpoints.

A generator is model knowledge (how weights concatenate, which tables are derived, which kernels a
layer calls); the engine holds none of it. Reference counterparts: tools/kern_manifest.py (normalize,
program helper), tools/once.py (load programs), tools/toy/gen.py:238-246 (safetensors writer).
"""
from __future__ import annotations

import json
import os
import struct
from pathlib import Path

import torch

# KERN_B200_CHECKED=1: the checked kernel build (its own directory, its own hashes in the manifests' module pins)
KERNELS_DIR = Path(__file__).resolve().parent.parent / ("kernels_checked" if os.environ.get("KERN_B200_CHECKED", "0") not in ("", "0") else "kernels")
SMS = 148                      # B200: the persistent kernels launch one CTA per SM
I64_MAX = (1 << 63) - 1
I32_MAX = (1 << 31) - 1
BM, BK = 128, 64
GEMM_STAGES = {256: 4, 128: 6, 64: 8, 32: 8}

_ST_DTYPES = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32", torch.int64: "I64",
              torch.int32: "I32", torch.uint8: "U8", torch.int8: "I8"}
if hasattr(torch, "float8_e4m3fn"):
    _ST_DTYPES[torch.float8_e4m3fn] = "F8_E4M3"


def kernel_index() -> dict:
    """sha256 pins of the in-tree cubins, written by the build."""
    from .. import _build

    _build.ensure_built()
    return json.loads((KERNELS_DIR / "index.json").read_text())


def modules_for(names) -> dict:
    idx = kernel_index()
    names = list(names)
    if "gemm_bf16" in names and "gemv_bf16" not in names:
        names.append("gemv_bf16")          # every gemm_op carries the weight-streaming launches for a handful of rows
    return {n: {"source": idx[n]["source"], "sha256": idx[n]["sha256"], "multicast": False} for n in names}


def ensure_modules(doc: dict) -> dict:
    """Add the built-in modules that some launch of `doc` names and `doc["modules"]` lacks."""
    idx = None
    for op in doc["ops"].values():
        for l in op.get("impl", {}).get("launches", []):
            m = l.get("module")
            if m and m not in doc["modules"]:
                idx = idx or kernel_index()
                if m in idx:
                    doc["modules"][m] = {"source": idx[m]["source"], "sha256": idx[m]["sha256"], "multicast": False}
    return doc


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """8-byte little-endian header length, JSON header padded to 8 bytes, raw little-endian data."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST_DTYPES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def read_safetensors(path) -> dict[str, torch.Tensor]:
    inv = {v: k for k, v in _ST_DTYPES.items()}
    data = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + hlen])
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        buf = bytearray(data[8 + hlen + lo:8 + hlen + hi])
        dt = inv[e["dtype"]]
        out[name] = torch.frombuffer(buf, dtype=dt).reshape(e["shape"]).clone() if hi > lo else torch.empty(e["shape"], dtype=dt)
    return out


def f64_bits(v: float) -> int:
    """A double passed through an 8-byte integer parameter slot."""
    return struct.unpack("<q", struct.pack("<d", float(v)))[0]


# ---- op builders: one place that knows each kernel's launch ABI ------------------------------------
GEMV_ROWS = 4


def gemm_smem(bn: int) -> int:
    return 1024 + GEMM_STAGES[bn] * (BM * BK * 2 + bn * BK * 2) + 256


def gemm_ranges(n: int, var_max: int, tiles=(256, 128, 64), sms: int = SMS):
    """`when` ranges of the row count -> N tile.

    Up to two M tiles (256 rows) the op is bound by streaming the weights, and what matters is how evenly the tiles
    cover the SMs: the tile width with the least `waves x width` (work of the slowest SM) wins, narrow tiles included.
    Beyond that it is tensor-core bound: the widest tile that still gives every SM a tile (256 once they fill every SM,
    128 from half the SMs on — a narrower tile feeds the tensor cores worse than a partly idle grid does)."""
    def cost(bn, m_tiles):
        t = m_tiles * -(-n // bn)
        return -(-t // sms) * bn * (1 + 8 / bn)      # a narrow tile pays more per byte (fewer bytes in flight, more tile turns)

    out, hi = [], var_max
    fill = {256: 1.0, 128: 0.5}
    for i, bn in enumerate(tiles):
        ncols = -(-n // bn)
        need_m_tiles = -(-int(sms * fill.get(bn, 1.0)) // ncols)
        lo = 1 if i == len(tiles) - 1 else (need_m_tiles - 1) * BM + 1
        lo = max(2 * BM + 1, lo)
        if lo <= hi:
            out.append((bn, lo, hi))
            hi = lo - 1
        if hi <= 2 * BM:
            break
    for m_tiles in (2, 1):
        lo, top = (m_tiles - 1) * BM + 1, min(m_tiles * BM, var_max)
        if lo > top:
            continue
        best = min([t for t in tiles if t >= 64], key=lambda bn: (cost(bn, m_tiles), -bn))   # 32-wide tiles measured slower here
        if out and out[-1][0] == best and out[-1][1] == top + 1:
            out[-1] = (best, lo, out[-1][2])
        else:
            out.append((best, lo, top))
    return out


M256_GAIN = 1.10     # measured speed of a 256-row tile over two 128-row tiles at large sizes (8192^3: 1532 vs 1318 TF; 0 turns them off)


def m256_split(n: int, lo: int, hi: int, sms: int = SMS):
    """Sub-ranges of [lo, hi] rows by tile height: 256 where `waves x tile work` is smaller than with 128-row tiles."""
    ncols = -(-n // 256)
    out = []
    r = lo
    while r <= hi:
        top = min(hi, -(-r // BM) * BM)            # rows up to the next multiple of 128 share their tile counts
        c256 = -(-(-(-top // 256) * ncols) // sms) * 2.0 / M256_GAIN
        c128 = -(-(-(-top // BM) * ncols) // sms) * 1.0
        bm = 256 if c256 < c128 else BM
        if out and out[-1][0] == bm:
            out[-1] = (bm, out[-1][1], top)
        else:
            out.append((bm, r, top))
        r = top + 1
    return out


def gemm_op(n: int, k: int, *, epilogue: str = "store", rows_var: str = "tokens", rows_max: int,
            lda: int | None = None, ldc: int | None = None) -> dict:
    """C[rows, n] = A[rows, k] · W[n, k]ᵀ through the tcgen05 GEMM, one launch per `when` range.

    Interface: [a, w, c, rows, err]. epilogue store | acc (c += …, c is inout) | f32 | swiglu
    (c is [rows, n/2] over weights stacked [gate rows ; up rows])."""
    lda = k if lda is None else lda
    out_cols = n // 2 if epilogue == "swiglu" else n
    ldc = out_cols if ldc is None else ldc
    cdt = "f32" if epilogue == "f32" else "bf16"
    cdir = "inout" if epilogue == "acc" else "out"
    suffix = {"store": "", "acc": "_acc", "f32": "_f32", "swiglu": "_swiglu"}[epilogue]
    iface = ["in buffer<bf16>", "in buffer<bf16>", f"{cdir} buffer<{cdt}>", "i32", "out buffer<i32>"]
    lparams = ["bytes<128>", "bytes<128>", f"{cdir} buffer<{cdt}>", "in buffer<bf16>", "i32", "i32", "i32", "i32",
               "out buffer<i32>"]
    launches = []
    # a handful of rows: the weight-streaming kernel (one launch per row-count class), above it the tensor-core tiles
    for mt, lo in ((1, 1), (2, 2), (4, 3)):
        hi = min(mt, rows_max)
        if lo > hi:
            continue
        when = {"var": rows_var}
        if lo > 1:
            when["min"] = lo
        if hi < rows_max:
            when["max"] = hi
        launch = {"module": "gemv_bf16", "entry": f"kern_gemv_bf16_tn{suffix}_m{mt}", "block": [256, 1, 1], "grid": [8 * SMS, 1, 1],
                  "params": ["in buffer<bf16>", "in buffer<bf16>", f"{cdir} buffer<{cdt}>", "in buffer<bf16>" if epilogue == "acc" else "i64",
                             "i32", "i32", "i32", "i32", "i32", "out buffer<i32>"],
                  "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 2} if epilogue == "acc" else {"i64": 0}, {"param": 3},
                           {"i32": n}, {"i32": k}, {"i32": lda}, {"i32": ldc}, {"param": 4}]}
        if len(when) > 1:
            launch["when"] = when
        launches.append(launch)
    tiles = (256, 128, 64, 32) if epilogue in ("store", "acc") else (256, 128, 64)
    ranges = []
    for bn, lo, hi in gemm_ranges(n, rows_max, tiles):
        if bn == 256 and epilogue in ("store", "acc", "swiglu") and M256_GAIN:
            ranges += [(bn, bm, a, b) for bm, a, b in m256_split(n, lo, hi)]
        else:
            ranges.append((bn, BM, lo, hi))
    for bn, bm, lo, hi in ranges:
        lo = max(lo, GEMV_ROWS + 1)
        if lo > hi:
            continue
        when = {"var": rows_var}
        if lo > 1:
            when["min"] = lo
        if hi < rows_max:
            when["max"] = hi
        launch = {
            "module": "gemm_bf16", "entry": f"kern_gemm_bf16_tn{suffix}{'_m256' if bm == 256 else ''}_n{bn}", "params": lparams,
            "block": [192, 1, 1], "grid": [SMS, 1, 1], "shared_mem": gemm_smem(bn),
            "args": [
                {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
                    "param": 0, "dtype": "bf16", "dims": [k, 0], "strides": [lda * 2], "box": [BK, bm],
                    "swizzle": 128, "l2_promotion": 256}}]}},
                {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
                    "param": 1, "dtype": "bf16", "dims": [k, n], "strides": [k * 2],
                    "box": [BK, bn // 2 if epilogue == "swiglu" else bn],
                    "swizzle": 128, "l2_promotion": 256}}]}},
                {"param": 2}, {"param": 2 if epilogue == "acc" else 0}, {"param": 3}, {"i32": n}, {"i32": k},
                {"i32": ldc}, {"param": 4}],
        }
        if len(when) > 1:
            launch["when"] = when
        launches.append(launch)
    return {"params": iface, "impl": {"launches": launches}}


AG_MAX_BLOCKS = 128      # 128-row blocks the fused all-gather GEMM keeps counters for (16 384 rows)


def ag_gemm_buffers(rows_max: int, k: int, nranks: int, group: str = "tp", alternate: bool = False) -> dict:
    """Buffers of the all-gather fused into the GEMM: `ag.g` holds all rows (this rank writes its slice, the kernel
    pulls the rest), the barrier's flags, and the arrival counters. `alternate`: a second row buffer `ag.g1`, for
    callers that switch buffers from call to call and so need no barrier after the GEMM."""
    second = {"ag.g1": {"dtype": "bf16", "shape": [rows_max, k], "kind": "carry", "export": True},
              "ag.g1_peers": {"dtype": "u64", "shape": [nranks], "kind": "peer", "of": "ag.g1", "group": group}} if alternate else {}
    return {**second,
            "ag.g": {"dtype": "bf16", "shape": [rows_max, k], "kind": "carry", "export": True},
            "ag.g_peers": {"dtype": "u64", "shape": [nranks], "kind": "peer", "of": "ag.g", "group": group},
            "ag.bar": {"dtype": "u32", "shape": [32], "kind": "carry", "export": True},
            "ag.bar_peers": {"dtype": "u64", "shape": [nranks], "kind": "peer", "of": "ag.bar", "group": group},
            "ag.bar_epoch": {"dtype": "u32", "shape": [1], "kind": "carry"},
            "ag.blocks": {"dtype": "u32", "shape": [AG_MAX_BLOCKS], "kind": "carry"},
            "ag.cta_epochs": {"dtype": "u32", "shape": [SMS], "kind": "carry"}}


def ag_gemm_op(n: int, k: int, nranks: int, group: str = "tp", bn: int = 256, timeout_ns: int = 2_000_000_000,
               closing_barrier: bool = True) -> dict:
    """C[rows, n] = G[rows, k] . W[n, k]^T with the all-gather of G's row slices inside the GEMM kernel.
    Interface [g, g_peers, w, c, bar, bar_peers, bar_epoch, blocks, cta_epochs, err, rows]. A cross-rank barrier runs
    first (every slice is complete before anyone pulls it); `closing_barrier` adds one after the GEMM so that the
    same `g` can be rewritten by the next call (a caller that alternates two buffers drops it)."""
    iface = ["inout buffer<bf16>", "in buffer<u64>", "in buffer<bf16>", "out buffer<bf16>", "inout buffer<u32>", "in buffer<u64>",
             "inout buffer<u32>", "inout buffer<u32>", "inout buffer<u32>", "out buffer<i32>", "i32"]
    barrier = {"module": "tp_allreduce_norm", "entry": "kern_peer_barrier", "block": [32, 1, 1], "grid": [1, 1, 1],
               "params": ["inout buffer<u32>", "in buffer<u64>", "inout buffer<u32>", "out buffer<i32>", "i32", "i32", "i64"],
               "args": [{"param": 4}, {"param": 5}, {"param": 6}, {"param": 9}, {"rank": group}, {"i32": nranks},
                        {"i64": timeout_ns}]}
    gemm = {"module": "ag_gemm", "entry": f"kern_ag_gemm_bf16_tn_n{bn}", "block": [320, 1, 1], "grid": [SMS, 1, 1],
            "shared_mem": gemm_smem(bn),
            "params": ["bytes<128>", "bytes<128>", "out buffer<bf16>", "i32", "i32", "i32", "i32", "out buffer<i32>",
                       "in buffer<u64>", "inout buffer<u32>", "inout buffer<u32>", "i32", "i32", "i32"],
            "args": [
                {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
                    "param": 0, "dtype": "bf16", "dims": [k, 0], "strides": [k * 2], "box": [BK, BM], "swizzle": 128,
                    "l2_promotion": 256}}]}},
                {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
                    "param": 2, "dtype": "bf16", "dims": [k, n], "strides": [k * 2], "box": [BK, bn], "swizzle": 128,
                    "l2_promotion": 256}}]}},
                {"param": 3}, {"param": 10}, {"i32": n}, {"i32": k}, {"i32": n}, {"param": 9}, {"param": 1}, {"param": 7},
                {"param": 8}, {"rank": group}, {"i32": nranks}, {"i32": AG_MAX_BLOCKS}]}
    return {"params": iface, "impl": {"launches": [barrier, gemm] + ([dict(barrier)] if closing_barrier else [])}}


def rms_norm_op(n: int, eps: float, plus_one: bool = False, rows_var: str = "tokens", x_stride: int | None = None) -> dict:
    """Interface [x, w, y]; one row per CTA. `x_stride`: elements between rows of x when they are columns of wider rows."""
    entry = "kern_rms_norm_bf16" if n <= 8192 else "kern_rms_norm_wide_bf16"
    return {"params": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>"],
            "impl": {"launches": [{
                "module": "norm_embed", "entry": entry, "block": [256, 1, 1], "grid": [rows_var, 1, 1],
                "params": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "i32", "i32", "i32", "i32", "f32", "i32"],
                "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"i32": I32_MAX}, {"i32": n}, {"i32": x_stride or n}, {"i32": n},
                         {"f32": eps}, {"i32": int(plus_one)}]}]}}


def embedding_op(hidden: int, vocab: int, ids_dtype: str = "i64") -> dict:
    """Interface [ids, table, out, err]."""
    return {"params": [f"in buffer<{ids_dtype}>", "in buffer<bf16>", "out buffer<bf16>", "out buffer<i32>"],
            "impl": {"launches": [{
                "module": "norm_embed", "entry": f"kern_embedding_{ids_dtype}_bf16",
                "block": [min(256, max(32, hidden // 8)), 1, 1], "grid": ["tokens", 1, 1],
                "params": [f"in buffer<{ids_dtype}>", "in buffer<bf16>", "out buffer<bf16>", "i32", "i32", "i32", "out buffer<i32>"],
                "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"i32": I32_MAX}, {"i32": hidden}, {"i32": vocab}, {"param": 3}]}]}}


def rope_append_op(hq: int, hk: int, d: int, rot: int, page_size: int, max_pos: int, eps: float,
                   qk_norm: bool, norm_plus_one: bool = False, row_stride: int | None = None) -> dict:
    """Interface [qkv, kv state, positions, slots, cos, sin, (q_norm, k_norm,) err]."""
    iface = ["inout buffer<bf16>", "inout state", "in buffer<i64>", "in buffer<i64>", "in buffer<f32>", "in buffer<f32>"]
    lp = list(iface)
    args = [{"param": i} for i in range(6)]
    if qk_norm:
        iface += ["in buffer<bf16>", "in buffer<bf16>"]
        lp += ["in buffer<bf16>", "in buffer<bf16>"]
        args += [{"param": 6}, {"param": 7}]
    else:
        lp += ["i64", "i64"]
        args += [{"i64": 0}, {"i64": 0}]
    iface.append("out buffer<i32>")
    lp += ["i32"] * 6 + ["f32", "i32", "i64", "i32", "i32", "out buffer<i32>"]
    args += [{"i32": I32_MAX}, {"i32": hq}, {"i32": hk}, {"i32": d}, {"i32": rot}, {"i32": page_size}, {"f32": eps},
             {"i32": int(norm_plus_one)}, {"i64": I64_MAX}, {"i32": max_pos},
             {"i32": row_stride or (hq + 2 * hk) * d}, {"param": len(iface) - 1}]
    return {"params": iface, "impl": {"launches": [{
        "module": "attn_prep", "entry": "kern_rope_kv_append_bf16", "block": [128, 1, 1], "grid": ["tokens", 1, 1],
        "shared_mem": 4 * d * 4, "params": lp, "args": args}]}}


def attn_smem(d: int, prefill: bool = False) -> int:
    stages = 2 if (prefill and d <= 128) else (3 if d >= 256 else 4)
    return 1024 + stages * (2 * 64 * d * 2) + 64 * (d + 8) * 2 + 256


_ATTN_LP = ["bytes<128>", "in buffer<bf16>", "out buffer<bf16>", "i64", "i64", "in buffer<i32>", "in buffer<i32>",
            "i64", "i64", "i64"] + ["i32"] * 10 + ["f32", "out buffer<i32>"]


def _kv_map(d: int, page_size: int, state_param: int) -> dict:
    return {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
        "param": state_param, "dtype": "bf16", "dims": [d, 0], "strides": [d * 2], "box": [64, min(page_size, 64)],
        "swizzle": 128, "l2_promotion": 256}}]}}


def attn_mode(hq: int, hk: int, d: int) -> str:
    """How a ragged call's attention runs (`KERN_B200_ATTN`, for A/B):
    `auto`    (default for head_dim 128) by the call's sequence count: up to `FMHA_SEQS` sequences — prompt chunks with few or
              no decode rows beside them, where the causal kernel is the whole cost — as `fmha2`, more as `ragged`;
    `ragged`  one launch, the mma.sync causal kernel's CTAs next to the token-parallel kernel's (head_dim 64 / 128);
    `fmha`    one launch, the tcgen05 causal kernel's CTAs (64-token KV tiles) next to the token-parallel kernel's (head_dim 128);
    `fmha2`   the tcgen05 causal kernel, then the token-parallel kernel (`KERN_B200_FMHA_TILE` = 64 | 128);
    `two`     the mma.sync causal kernel, then the token-parallel kernel.
    `KERN_B200_FMHA=1` reads as `fmha`, `KERN_B200_ATTN_RAGGED=0` as `two`."""
    import os

    mode = os.environ.get("KERN_B200_ATTN")
    if mode is None:
        mode = "fmha" if os.environ.get("KERN_B200_FMHA", "0") == "1" else ("two" if os.environ.get("KERN_B200_ATTN_RAGGED", "1") == "0" else "auto")
    if mode in ("auto", "fmha", "fmha2") and not (d == 128 and 128 % (hq // hk) == 0):
        mode = "ragged"
    if mode == "ragged" and d not in (64, 128):
        mode = "two"
    if mode not in ("auto", "ragged", "fmha", "fmha2", "two"):
        raise ValueError(f"KERN_B200_ATTN={mode!r}: expected auto, ragged, fmha, fmha2 or two")
    return mode


FMHA_SEQS = 8      # `auto`: calls of up to this many sequences take the tcgen05 causal kernel


def fmha_prefill(hq: int, hk: int, d: int) -> bool:
    """Whether every ragged call's many-row list goes to the tcgen05 kernel (attn_fmha.cu), whose blocks are 128 rows."""
    return attn_mode(hq, hk, d) in ("fmha", "fmha2")


def attn_ragged(d: int) -> bool:
    """Whether head_dim `d` has a one-launch form of the ragged call."""
    return d in (64, 128)


def attn_prefill_op(hq: int, hk: int, d: int, page_size: int, table_width: int, q_stride: int) -> dict:
    """Ragged causal attention over the paged context.
    Interface [q(kv) buffer, kv state, out, block_table, seq_lens, cu_seqlens, work, work_count, err]."""
    g = hq // hk
    mode = attn_mode(hq, hk, d)
    if mode == "auto":
        # few sequences: the tcgen05 causal kernel, then the token-parallel kernel for whatever decode rows there are;
        # many: the one-launch form whose decode CTAs stream KV next to the mma.sync prompt CTAs
        import os

        few = {"var": "seqs", "max": FMHA_SEQS}
        saved = os.environ.get("KERN_B200_ATTN")
        try:
            os.environ["KERN_B200_ATTN"] = "fmha2"
            a = attn_prefill_op(hq, hk, d, page_size, table_width, q_stride)
            os.environ["KERN_B200_ATTN"] = "ragged"
            b = attn_prefill_op(hq, hk, d, page_size, table_width, q_stride)
        finally:
            if saved is None:
                os.environ.pop("KERN_B200_ATTN", None)
            else:
                os.environ["KERN_B200_ATTN"] = saved
        launches = [dict(l, when=few) for l in a["impl"]["launches"]] + \
                   [dict(l, when={"var": "seqs", "min": FMHA_SEQS + 1}) for l in b["impl"]["launches"]]
        return {"params": a["params"], "impl": {"launches": launches}}
    fmha = mode in ("fmha", "fmha2")
    tpb = (128 if fmha else 64) // g
    iface = ["in buffer<bf16>", "in state", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "in buffer<i32>",
             "in buffer<i32>", "in buffer<i32>", "out buffer<i32>"]
    lp = list(_ATTN_LP)
    lp[7], lp[8], lp[9] = "in buffer<i32>", "in buffer<i32>", "in buffer<i32>"
    iface += ["in buffer<i32>", "in buffer<i32>"]     # the second work list (few-row sequences) and its count

    def args(work: int, count: int) -> list:
        return [_kv_map(d, page_size, 1), {"param": 0}, {"param": 2}, {"i64": 0}, {"i64": 0}, {"param": 3}, {"param": 4},
                {"param": 5}, {"param": work}, {"param": count}, {"i32": I32_MAX}, {"i32": hq}, {"i32": hk},
                {"i32": q_stride}, {"i32": hq * d}, {"i32": table_width}, {"i32": page_size}, {"i32": 1}, {"i32": 1},
                {"i32": I32_MAX}, {"f32": (d ** -0.5) * 1.4426950408889634}, {"param": 8}]

    # many-row sequences: row-parallel causal kernel (on the 5th-generation tensor cores for head_dim 128); few-row
    # sequences (decode rows riding in the ragged call): token-parallel kernel, so their KV streams at full bandwidth
    ragged_params = ["bytes<128>", "in buffer<bf16>", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "in buffer<i32>",
                     "in buffer<i32>", "in buffer<i32>", "in buffer<i32>", "in buffer<i32>"] + ["i32"] * 7 + ["f32", "out buffer<i32>"]
    ragged_args = [_kv_map(d, page_size, 1), {"param": 0}, {"param": 2}, {"param": 3}, {"param": 4}, {"param": 5}, {"param": 6},
                   {"param": 7}, {"param": 9}, {"param": 10}, {"i32": hq}, {"i32": hk}, {"i32": q_stride}, {"i32": hq * d},
                   {"i32": table_width}, {"i32": page_size}, {"i32": I32_MAX}, {"f32": (d ** -0.5) * 1.4426950408889634},
                   {"param": 8}]
    if mode == "fmha":
        # both lists in one launch, the prompt rows on the 5th-generation tensor cores: a tcgen05 CTA (64-token KV tiles,
        # 113 KB, 256 TMEM columns) and a token-parallel CTA share an SM
        return {"params": iface, "impl": {"launches": [{
            "module": "attn_fmha", "entry": "kern_attn_ragged_fmha_d128", "block": [192, 1, 1],
            "grid": [hk, {"add": [{"ceil_div": ["tokens", tpb]}, "seqs"]}, 1],
            "shared_mem": 768 + 128 * d * 2 + 128 * 64 * 2 + 2 * 2 * (64 * d * 2) + 256,
            "params": ragged_params, "args": ragged_args}]}}
    if mode == "fmha2":
        import os

        tile = int(os.environ.get("KERN_B200_FMHA_TILE", "64"))      # tokens per KV tile: 64 (two CTAs per SM) or 128
        many = {"module": "attn_fmha", "entry": "kern_attn_fmha_prefill_d128" + ("_t64" if tile == 64 else ""), "block": [192, 1, 1],
                "grid": [hk, {"add": [{"ceil_div": ["tokens", tpb]}, "seqs"]}, 1],
                "shared_mem": (768 if tile == 64 else 1024) + 128 * d * 2 + 128 * tile * 2 + 2 * 2 * (tile * d * 2) + 256,
                "params": ["bytes<128>", "in buffer<bf16>", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "in buffer<i32>",
                           "in buffer<i32>", "in buffer<i32>"] + ["i32"] * 7 + ["f32", "out buffer<i32>"],
                "args": [_kv_map(d, page_size, 1), {"param": 0}, {"param": 2}, {"param": 3}, {"param": 4}, {"param": 5}, {"param": 6},
                         {"param": 7}, {"i32": hq}, {"i32": hk}, {"i32": q_stride}, {"i32": hq * d}, {"i32": table_width},
                         {"i32": page_size}, {"i32": I32_MAX}, {"f32": (d ** -0.5) * 1.4426950408889634}, {"param": 8}]}
    elif mode == "ragged":
        # both lists in one launch: the two kernels' CTAs alternate, two per SM, so the decode rows' KV streams under
        # the prompt rows' tensor-core work (a sequence is on one list only, so the grid bound is unchanged)
        return {"params": iface, "impl": {"launches": [{
            "module": "attn_paged", "entry": f"kern_attn_ragged_paged_d{d}", "block": [160, 1, 1],
            "grid": [hk, {"add": [{"ceil_div": ["tokens", tpb]}, "seqs"]}, 1], "shared_mem": attn_smem(d, prefill=True),
            "params": ragged_params, "args": ragged_args}]}}
    else:
        many = {"module": "attn_paged", "entry": f"kern_attn_prefill_paged_d{d}", "block": [160, 1, 1],
                "grid": [hk, {"add": [{"ceil_div": ["tokens", tpb]}, "seqs"]}, 1], "shared_mem": attn_smem(d, prefill=True),
                "params": lp, "args": args(6, 7)}
    return {"params": iface, "impl": {"launches": [
        many,
        {"module": "attn_paged", "entry": f"kern_attn_decode_paged_d{d}", "block": [160, 1, 1],
         "grid": [hk, "seqs", 1], "shared_mem": attn_smem(d), "params": lp, "args": args(9, 10)}]}}


def attn_decode_dcp_op(hq: int, hk: int, d: int, page_size: int, table_width: int, q_stride: int, world: int,
                       group: str = "dcp", splits: int = 4) -> dict:
    """Decode attention of a member of a by-position (context-parallel) group: positions are dealt round-robin, the
    member attends over its own pages and leaves un-normalised partials, the group all-gathers them and every member
    merges (log-sum-exp) to the same rows.
    Interface [q(kv) buffer, kv state, out, block_table, seq_lens (whole lengths), err, count_o, count_ml, rows_hq, seqs]:
    the call passes `hq * splits * d`, `hq * splits * 2` and `hq` times `seqs` and `seqs` itself."""
    iface = ["in buffer<bf16>", "in state", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "out buffer<i32>",
             "i64", "i64", "i32", "i32"]
    scratch = {"local_lens": {"dtype": "i32", "shape": ["seqs"]},
               "ws_o": {"dtype": "f32", "shape": ["seqs", hq * splits * d]}, "ws_ml": {"dtype": "f32", "shape": ["seqs", hq * splits * 2]},
               "all_o": {"dtype": "f32", "shape": ["seqs", world * hq * splits * d]},
               "all_ml": {"dtype": "f32", "shape": ["seqs", world * hq * splits * 2]}}
    prepare = {"module": "attn_paged", "entry": "kern_dcp_prepare", "block": [128, 1, 1], "grid": ["seqs", 1, 1],
               "params": ["in buffer<i32>", "out buffer<i32>", "out buffer<f32>", "i32", "i32", "i32", "i32"],
               "args": [{"param": 4}, {"scratch": "local_lens"}, {"scratch": "ws_ml"}, {"param": 9}, {"rank": group},
                        {"i32": world}, {"i32": hq * splits}]}
    lp = list(_ATTN_LP)
    lp[3], lp[4] = "out buffer<f32>", "inout buffer<f32>"
    lp[6] = "in buffer<i32>"
    g = hq // hk
    nblk = -(-1 // max(1, 16 // g))
    attn = {"module": "attn_paged", "entry": f"kern_attn_decode_paged_d{d}", "block": [160, 1, 1],
            "grid": [hk * nblk, "seqs", splits], "shared_mem": attn_smem(d), "params": lp,
            "args": [_kv_map(d, page_size, 1), {"param": 0}, {"param": 2}, {"scratch": "ws_o"}, {"scratch": "ws_ml"}, {"param": 3},
                     {"scratch": "local_lens"}, {"i64": 0}, {"i64": 0}, {"i64": 0}, {"i32": I32_MAX}, {"i32": hq}, {"i32": hk},
                     {"i32": q_stride}, {"i32": hq * d}, {"i32": table_width}, {"i32": page_size}, {"i32": 1},
                     {"i32": splits | (splits << 16)}, {"i32": I32_MAX}, {"f32": (d ** -0.5) * 1.4426950408889634}, {"param": 5}]}
    gather = lambda src, dst, cnt: {"entry": "extern:nccl_allgather_f32", "params": ["in buffer<f32>", "out buffer<f32>", "i64", "i32"],
                                    "args": [{"scratch": src}, {"scratch": dst}, {"param": cnt}, {"rank": group}]}
    merge = {"module": "attn_paged", "entry": "kern_attn_merge_ranks", "block": [min(256, d), 1, 1],
             "grid": [{"mul": ["seqs", hq]}, 1, 1],
             "params": ["in buffer<f32>", "in buffer<f32>", "out buffer<bf16>", "i32", "i32", "i32", "i32", "i32", "i32"],
             "args": [{"scratch": "all_o"}, {"scratch": "all_ml"}, {"param": 2}, {"param": 8}, {"i32": hq}, {"i32": d},
                      {"i32": splits}, {"i32": world}, {"i32": hq * d}]}
    return {"params": iface, "impl": {"launches": [prepare, attn, gather("ws_o", "all_o", 6), gather("ws_ml", "all_ml", 7), merge],
                                      "scratch": scratch}}


def attn_plan_op(hq: int, hk: int, seqs_max: int, d: int = 0) -> dict:
    """Interface [cu_seqlens, work, work_count, seqs, max_items]; the attention grid's (sequence, block)
    work list. A call passes ``{"var": "seqs"}`` and ``attn_plan_items(...)``. `d`: the head_dim, which decides the
    block of the many-row list (the tcgen05 kernel's tile is 128 rows)."""
    g = hq // hk
    tpd = max(1, 16 // g)
    mode = attn_mode(hq, hk, d)

    def plan(tpb: int, when: dict | None) -> dict:
        l = {"module": "attn_paged", "entry": "kern_attn_plan", "block": [256, 1, 1], "grid": [1, 1, 1],
             "params": ["in buffer<i32>", "i32", "i32", "i32", "i32", "out buffer<i32>", "out buffer<i32>", "i32",
                        "out buffer<i32>", "out buffer<i32>", "i32"],
             "args": [{"param": 0}, {"param": 3}, {"i32": tpb}, {"i32": tpd}, {"i32": tpd}, {"param": 1}, {"param": 2},
                      {"param": 4}, {"param": 5}, {"param": 6}, {"param": 3}]}
        if when:
            l["when"] = when
        return l

    if mode == "auto" and seqs_max > FMHA_SEQS:
        # the many-row list in blocks of the kernel that will read it: 128 rows for the tcgen05 kernel (few sequences),
        # 64 for the mma.sync kernel
        launches = [plan(128 // g, {"var": "seqs", "max": FMHA_SEQS}), plan(64 // g, {"var": "seqs", "min": FMHA_SEQS + 1})]
    else:
        launches = [plan((128 if mode in ("auto", "fmha", "fmha2") else 64) // g, None)]
    return {"params": ["in buffer<i32>", "out buffer<i32>", "out buffer<i32>", "i32", "i32", "out buffer<i32>", "out buffer<i32>"],
            "impl": {"launches": launches}}


def attn_plan_items(hq: int, hk: int) -> dict:
    """Expression for the most work items a call can have: one per block of rows plus one per sequence."""
    return {"add": [{"ceil_div": ["tokens", 64 // (hq // hk)]}, "seqs"]}


def attn_decode_op(hq: int, hk: int, d: int, page_size: int, table_width: int, q_stride: int, seqs_max: int,
                   rows: int = 1, sms: int = SMS) -> dict:
    """Decode / verify rows over the paged context, split-KV chosen by `when` ranges of the batch.
    Interface [q(kv) buffer, kv state, out, block_table, seq_lens, err]."""
    g = hq // hk
    nblk = -(-rows // max(1, 16 // g))
    iface = ["in buffer<bf16>", "in state", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "out buffer<i32>"]
    ranges, hi = [], seqs_max
    for splits in (1, 2, 4, 8, 16, 32):
        # enough sequences that hk * nblk * seqs * splits covers the SMs
        lo = max(1, -(-sms // (hk * nblk * splits)))
        if splits == 32:
            lo = 1
        if lo <= hi:
            ranges.append((splits, lo, hi))
            hi = lo - 1
        if hi < 1:
            break
    launches, scratch = [], {}
    max_splits = max(s for s, _, _ in ranges)
    if max_splits > 1:
        scratch = {"ws_o": {"dtype": "f32", "shape": ["tokens", hq * max_splits * d]},
                   "ws_ml": {"dtype": "f32", "shape": ["tokens", hq * max_splits * 2]}}
    for splits, lo, hi in ranges:
        when = {"var": "seqs"}
        if lo > 1:
            when["min"] = lo
        if hi < seqs_max:
            when["max"] = hi
        lp = list(_ATTN_LP)
        ws = [{"i64": 0}, {"i64": 0}]
        if splits > 1:
            lp[3], lp[4] = "out buffer<f32>", "out buffer<f32>"
            ws = [{"scratch": "ws_o"}, {"scratch": "ws_ml"}]
        args = [_kv_map(d, page_size, 1), {"param": 0}, {"param": 2}, *ws, {"param": 3}, {"param": 4}, {"i64": 0},
                {"i64": 0}, {"i64": 0}, {"i32": I32_MAX}, {"i32": hq}, {"i32": hk}, {"i32": q_stride}, {"i32": hq * d},
                {"i32": table_width}, {"i32": page_size}, {"i32": rows}, {"i32": splits}, {"i32": I32_MAX},
                {"f32": (d ** -0.5) * 1.4426950408889634}, {"param": 5}]
        launch = {"module": "attn_paged", "entry": f"kern_attn_decode_paged_d{d}", "block": [160, 1, 1],
                  "grid": [hk * nblk, "seqs", splits], "shared_mem": attn_smem(d), "params": lp, "args": args}
        if len(when) > 1:
            launch["when"] = when
        launches.append(launch)
        if splits > 1:
            merge = {"module": "attn_paged", "entry": "kern_attn_merge_splits", "block": [min(256, d), 1, 1],
                     "grid": [{"mul": ["tokens", hq]}, 1, 1],
                     "params": ["in buffer<f32>", "in buffer<f32>", "out buffer<bf16>", "i32", "i32", "i32", "i32", "i32"],
                     "args": [{"scratch": "ws_o"}, {"scratch": "ws_ml"}, {"param": 2}, {"i32": I32_MAX}, {"i32": hq},
                              {"i32": d}, {"i32": splits}, {"i32": hq * d}]}
            if len(when) > 1:
                merge["when"] = when
            launches.append(merge)
    impl = {"launches": launches}
    if scratch:
        impl["scratch"] = scratch
    return {"params": iface, "impl": impl}


def last_row_op(row_bytes: int) -> dict:
    """Interface [src, dst, cu_seqlens]: the last row of every sequence of a ragged batch."""
    return {"params": ["in buffer<bf16>", "out buffer<bf16>", "in buffer<i32>"], "impl": {"launches": [{
        "module": "misc", "entry": "kern_last_row", "block": [128, 1, 1], "grid": ["seqs", 1, 1],
        "params": ["in buffer<bf16>", "out buffer<bf16>", "in buffer<i32>", "i32", "i32"],
        "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"i32": I32_MAX}, {"i32": row_bytes}]}]}}


def argmax_op(vocab: int, dtype: str = "bf16", parts: int = 32, rows_var: str = "seqs") -> dict:
    """Interface [logits, tokens out]."""
    return {"params": [f"in buffer<{dtype}>", "out buffer<i64>"], "impl": {
        "scratch": {"pv": {"dtype": "f32", "shape": [rows_var, parts]}, "pi": {"dtype": "i32", "shape": [rows_var, parts]}},
        "launches": [
            {"module": "sampling", "entry": f"kern_argmax_partial_{dtype}", "block": [256, 1, 1], "grid": [rows_var, parts, 1],
             "params": [f"in buffer<{dtype}>", "out buffer<f32>", "out buffer<i32>", "i32", "i32", "i32"],
             "args": [{"param": 0}, {"scratch": "pv"}, {"scratch": "pi"}, {"i32": I32_MAX}, {"i32": vocab}, {"i32": vocab}]},
            {"module": "sampling", "entry": "kern_argmax_final_i64", "block": [32, 1, 1], "grid": [rows_var, 1, 1],
             "params": ["in buffer<f32>", "in buffer<i32>", "out buffer<i64>", "i32", "i32"],
             "args": [{"scratch": "pv"}, {"scratch": "pi"}, {"param": 1}, {"i32": I32_MAX}, {"i32": parts}]}]}}


def sample_op(vocab: int, dtype: str = "bf16") -> dict:
    """Interface [logits, tokens out, temperature, top_k, top_p, min_p, seed, seq_lens (draw offset)]."""
    return {"params": [f"in buffer<{dtype}>", "out buffer<i64>", "in buffer<f32>", "in buffer<i32>", "in buffer<f32>",
                       "in buffer<f32>", "in buffer<i64>", "in buffer<i32>"],
            "impl": {"scratch": {"probs": {"dtype": "f32", "shape": ["seqs", vocab]}},
                     "launches": [{"module": "sampling", "entry": f"kern_sample_{dtype}", "block": [1024, 1, 1],
                                   "grid": ["seqs", 1, 1],
                                   "params": [f"in buffer<{dtype}>", "out buffer<f32>", "out buffer<i64>", "in buffer<f32>",
                                              "in buffer<i32>", "in buffer<f32>", "in buffer<f32>", "in buffer<i64>",
                                              "in buffer<i32>", "i32", "i32", "i32"],
                                   "args": [{"param": 0}, {"scratch": "probs"}, {"param": 1}, {"param": 2}, {"param": 3},
                                            {"param": 4}, {"param": 5}, {"param": 6}, {"param": 7}, {"i32": I32_MAX},
                                            {"i32": vocab}, {"i32": vocab}]}]}}


def rope_table_op(max_pos: int, rot: int, theta: float) -> dict:
    """Interface [cos, sin]: the `once` program's table of angles."""
    return {"params": ["out buffer<f32>", "out buffer<f32>"], "impl": {"launches": [{
        "module": "attn_prep", "entry": "kern_rope_table_f32", "block": [256, 1, 1],
        "grid": [min(1024, -(-max_pos * (rot // 2) // 256)), 1, 1],
        "params": ["out buffer<f32>", "out buffer<f32>", "i32", "i32", "i64"],
        "args": [{"param": 0}, {"param": 1}, {"i32": max_pos}, {"i32": rot}, {"i64": f64_bits(theta)}]}]}}


# ---- tensor-parallel ops ---------------------------------------------------------------------------
TP_GRID = 592                      # most CTAs of the fused all-reduce (4 per SM) = columns of its flag arrays
TP_ONESHOT_ROWS = 64               # up to this many rows every rank reduces everything itself


def tp_slot_rows(rows_max: int, nranks: int, grid: int = TP_GRID) -> int:
    """Rows one staging slot must hold: all rows in one-shot mode, a rank's dealt share in two-shot."""
    per_cta = -(-rows_max // grid)
    return max(TP_ONESHOT_ROWS, -(-per_cta // nranks) * grid)


def tp_allreduce_norm_op(hidden: int, eps: float, nranks: int, rows_max: int, group: str = "tp",
                         plus_one: bool = False, timeout_ns: int = 2_000_000_000, fused_gemm: bool = False,
                         lamport: bool = False) -> dict:
    """x += sum over the group of `partial`; xn = rmsnorm(x) * w — one kernel over NVLink peer memory.
    `fused_gemm`: above TP_ONESHOT_ROWS rows the partials were already pushed by tp_gemm_reduce_op's epilogue.
    `lamport`: up to TP_ONESHOT_ROWS rows use the flagless one-shot; the interface grows by [lamport, lamport_peers,
    lamport_epochs] (buffers of `tp_buffers(..., lamport=True)`, poisoned once by `tp_lamport_init_op`).
    Interface [partial, x, x_peers, xn, w, comm, comm_peers, flags, flag_peers, epochs, err, rows]."""
    slot_rows = tp_slot_rows(rows_max, nranks)
    iface = ["in buffer<bf16>", "inout buffer<bf16>", "in buffer<u64>", "out buffer<bf16>", "in buffer<bf16>",
             "inout buffer<bf16>", "in buffer<u64>", "inout buffer<u32>", "in buffer<u64>", "inout buffer<u32>",
             "out buffer<i32>", "i32"]
    lp = iface[:11] + ["i32", "i32", "i32", "i32", "i32", "f32", "i32", "i32", "i64", "i32"]
    launches = []
    # few rows: one-shot on a grid no larger than the rows (every CTA of the grid exchanges flags);
    # many rows: two-shot on the full grid
    if lamport:
        # few rows: the flagless one-shot (payload is its own arrival signal), one CTA per row
        iface += ["inout buffer<bf16>", "in buffer<u64>", "inout buffer<u32>"]
        when = {"var": "tokens"}
        if rows_max > TP_ONESHOT_ROWS:
            when["max"] = TP_ONESHOT_ROWS
        launch = {"module": "tp_allreduce_norm", "entry": "kern_tp_allreduce_lamport", "block": [256, 1, 1],
                  "grid": ["tokens", 1, 1], "shared_mem": hidden * 4,
                  "params": ["in buffer<bf16>", "inout buffer<bf16>", "out buffer<bf16>", "in buffer<bf16>", "inout buffer<bf16>",
                             "in buffer<u64>", "inout buffer<u32>", "out buffer<i32>", "i32", "i32", "i32", "i32", "i32", "f32",
                             "i32", "i64"],
                  "args": [{"param": 0}, {"param": 1}, {"param": 3}, {"param": 4}, {"param": 12}, {"param": 13}, {"param": 14},
                           {"param": 10}, {"rank": group}, {"i32": nranks}, {"param": 11}, {"i32": hidden},
                           {"i32": TP_ONESHOT_ROWS}, {"f32": eps}, {"i32": int(plus_one)}, {"i64": timeout_ns}]}
        if len(when) > 1:
            launch["when"] = when
        launches.append(launch)
    for mode, grid, lo, hi in ((0, 16, 1, min(16, rows_max)), (0, TP_ONESHOT_ROWS, 17, min(TP_ONESHOT_ROWS, rows_max)),
                               (2 if fused_gemm else 1, TP_GRID, TP_ONESHOT_ROWS + 1, rows_max)):
        if lamport and mode == 0:
            continue
        if lo > hi:
            continue
        when = {"var": "tokens"}
        if lo > 1:
            when["min"] = lo
        if hi < rows_max:
            when["max"] = hi
        launch = {"module": "tp_allreduce_norm", "entry": "kern_tp_allreduce_residual_norm", "block": [256, 1, 1],
                  "grid": [grid, 1, 1], "shared_mem": hidden * 4, "params": lp,
                  "args": [{"param": i} for i in range(11)] + [{"rank": group}, {"i32": nranks}, {"param": 11}, {"i32": hidden},
                                                                {"i32": slot_rows}, {"f32": eps}, {"i32": int(plus_one)},
                                                                {"i32": mode}, {"i64": timeout_ns}, {"i32": TP_GRID}]}
        if len(when) > 1:
            launch["when"] = when
        launches.append(launch)
    return {"params": iface, "impl": {"launches": launches}}


def tp_gemm_reduce_op(n: int, k: int, nranks: int, rows_max: int, group: str = "tp") -> dict:
    """A tensor-parallel partial GEMM feeding the fused all-reduce. Up to TP_ONESHOT_ROWS rows it stores the partial
    (the one-shot all-reduce pushes it); above, its epilogue pushes every row over NVLink straight into the reducing
    rank's staging slot, and the all-reduce runs in mode 2 (reduce + residual + norm + gather only).
    Interface [a, w, part, comm_peers, epochs, rows, err]."""
    slot_rows = tp_slot_rows(rows_max, nranks)
    iface = ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "in buffer<u64>", "in buffer<u32>", "i32", "out buffer<i32>"]
    a_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
        "param": 0, "dtype": "bf16", "dims": [k, 0], "strides": [k * 2], "box": [BK, BM], "swizzle": 128, "l2_promotion": 256}}]}}
    b_map = lambda bn: {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
        "param": 1, "dtype": "bf16", "dims": [k, n], "strides": [k * 2], "box": [BK, bn], "swizzle": 128, "l2_promotion": 256}}]}}
    launches = []
    small = min(TP_ONESHOT_ROWS, rows_max)
    for bn, lo, hi in gemm_ranges(n, small):
        when = {"var": "tokens", "max": hi}
        if lo > 1:
            when["min"] = lo
        launches.append({"module": "gemm_bf16", "entry": f"kern_gemm_bf16_tn_n{bn}", "block": [192, 1, 1], "grid": [SMS, 1, 1],
                         "shared_mem": gemm_smem(bn), "when": when,
                         "params": ["bytes<128>", "bytes<128>", "out buffer<bf16>", "i64", "i32", "i32", "i32", "i32", "out buffer<i32>"],
                         "args": [a_map, b_map(bn), {"param": 2}, {"i64": 0}, {"param": 5}, {"i32": n}, {"i32": k}, {"i32": n},
                                  {"param": 6}]})
    for bn, lo, hi in gemm_ranges(n, rows_max):
        lo = max(lo, small + 1)
        if lo > hi:
            continue
        when = {"var": "tokens", "min": lo}
        if hi < rows_max:
            when["max"] = hi
        launches.append({"module": "tp_gemm", "entry": f"kern_tp_gemm_scatter_bf16_n{bn}", "block": [192, 1, 1], "grid": [SMS, 1, 1],
                         "shared_mem": gemm_smem(bn) + 20480, "when": when,     # + the epilogue's row staging
                         "params": ["bytes<128>", "bytes<128>", "i32", "i32", "i32", "out buffer<i32>", "in buffer<u64>",
                                    "in buffer<u32>", "i32", "i32", "i32", "i32"],
                         "args": [a_map, b_map(bn), {"param": 5}, {"i32": n}, {"i32": k}, {"param": 6}, {"param": 3}, {"param": 4},
                                  {"rank": group}, {"i32": nranks}, {"i32": TP_GRID}, {"i32": slot_rows}]})
    return {"params": iface, "impl": {"launches": launches}}


# ---- sequence-parallel layout inside a tensor-parallel group -----------------------------------------
SP_SUB = 32                        # rows per ownership sub-block: sub-block s belongs to rank s % nranks
SP_GRID = 2 * SMS                  # CTAs of the reduce + norm kernel
SP_FLAG_STRIDE = 32                # words per row of `sp.flags`


def sp_slot_rows(rows_max: int, nranks: int) -> int:
    """Rows one staging slot holds: a rank's share of the sub-blocks of the largest call."""
    return -(-(-(-rows_max // SP_SUB)) // nranks) * SP_SUB


def sp_buffers(hidden: int, nranks: int, rows_max: int, group: str = "tp") -> dict:
    """Exported buffers of the sequence-parallel path: staging slots the peers' GEMM epilogues push into, the
    all-gather buffer `sp.g` of normed rows, the two rows of epoch flags, and the local counters."""
    peer = lambda of: {"dtype": "u64", "shape": [nranks], "kind": "peer", "of": of, "group": group}
    return {
        "sp.comm": {"dtype": "bf16", "shape": [2, nranks, sp_slot_rows(rows_max, nranks), hidden], "kind": "carry", "export": True},
        "sp.comm_peers": peer("sp.comm"),
        "sp.flags": {"dtype": "u32", "shape": [2, SP_FLAG_STRIDE], "kind": "carry", "export": True},
        "sp.flags_peers": peer("sp.flags"),
        "sp.state": {"dtype": "u32", "shape": [2], "kind": "carry"},
        "sp.g": {"dtype": "bf16", "shape": [rows_max, hidden], "kind": "carry", "export": True},
        "sp.g_peers": peer("sp.g"),
        "sp.blocks": {"dtype": "u32", "shape": [AG_MAX_BLOCKS], "kind": "carry"},
        "sp.cta_epochs": {"dtype": "u32", "shape": [SMS], "kind": "carry"},
    }


def _when(var: str, lo: int, hi: int, var_max: int) -> dict | None:
    w = {"var": var}
    if lo > 1:
        w["min"] = lo
    if hi < var_max:
        w["max"] = hi
    return w if len(w) > 1 else None


def sp_gemm_scatter_op(n: int, k: int, nranks: int, rows_max: int, group: str = "tp") -> dict:
    """A tensor-parallel partial GEMM whose epilogue is the push half of a reduce-scatter: every row of every tile goes
    from TMEM over NVLink into its owner's staging slot (sub-block ownership). `sp_reduce_norm_op` finishes it.
    Interface [a, w, comm_peers, state, rows, err]."""
    slot_rows = sp_slot_rows(rows_max, nranks)
    iface = ["in buffer<bf16>", "in buffer<bf16>", "in buffer<u64>", "in buffer<u32>", "i32", "out buffer<i32>"]
    a_map = {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
        "param": 0, "dtype": "bf16", "dims": [k, 0], "strides": [k * 2], "box": [BK, BM], "swizzle": 128, "l2_promotion": 256}}]}}
    b_map = lambda bn: {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
        "param": 1, "dtype": "bf16", "dims": [k, n], "strides": [k * 2], "box": [BK, bn], "swizzle": 128, "l2_promotion": 256}}]}}
    launches = []
    for bn, lo, hi in gemm_ranges(n, rows_max):
        launch = {"module": "tp_gemm", "entry": f"kern_tp_gemm_scatter_bf16_n{bn}", "block": [192, 1, 1], "grid": [SMS, 1, 1],
                  "shared_mem": gemm_smem(bn) + 20480,     # + the epilogue's row staging
                  "params": ["bytes<128>", "bytes<128>", "i32", "i32", "i32", "out buffer<i32>", "in buffer<u64>",
                             "in buffer<u32>", "i32", "i32", "i32", "i32"],
                  "args": [a_map, b_map(bn), {"param": 4}, {"i32": n}, {"i32": k}, {"param": 5}, {"param": 2}, {"param": 3},
                           {"rank": group}, {"i32": nranks}, {"i32": 0}, {"i32": slot_rows}]}
        w = _when("tokens", lo, hi, rows_max)
        if w:
            launch["when"] = w
        launches.append(launch)
    return {"params": iface, "impl": {"launches": launches}}


def sp_reduce_norm_op(hidden: int, eps: float, nranks: int, rows_max: int, group: str = "tp", plus_one: bool = False,
                      timeout_ns: int = 2_000_000_000, push: bool = True) -> dict:
    """On the rows this rank owns: x += sum of the partials the peers pushed; g = rmsnorm(x) * w. One kernel; it also
    lines the ranks up (bounded waits on epoch flags). `push`: the normed rows go straight into every rank's g (the
    all-gather as posted peer stores); off, they stay here and the next GEMM pulls them.
    Interface [x, g, w, comm, flags, flags_peers, state, err, rows, g_peers]."""
    iface = ["inout buffer<bf16>", "inout buffer<bf16>", "in buffer<bf16>", "inout buffer<bf16>", "inout buffer<u32>",
             "in buffer<u64>", "inout buffer<u32>", "out buffer<i32>", "i32", "in buffer<u64>"]      # comm is inout: the peers write it
    return {"params": iface, "impl": {"launches": [{
        "module": "tp_sp", "entry": "kern_sp_reduce_norm", "block": [256, 1, 1], "grid": [SP_GRID, 1, 1],
        "params": iface[:8] + ["i32", "i32", "i32", "i32", "i32", "f32", "i32", "i64", "in buffer<u64>" if push else "i64"],
        "args": [{"param": i} for i in range(8)] + [{"rank": group}, {"i32": nranks}, {"param": 8}, {"i32": hidden},
                                                     {"i32": sp_slot_rows(rows_max, nranks)}, {"f32": eps}, {"i32": int(plus_one)},
                                                     {"i64": timeout_ns}, {"param": 9} if push else {"i64": 0}]}]}}


def sp_ag_gemm_op(n: int, k: int, nranks: int, rows_max: int, group: str = "tp", epilogue: str = "store",
                  timeout_ns: int = 2_000_000_000, pushed: bool = True) -> dict:
    """C[rows, n] = G[rows, k] . W[n, k]^T where G's rows sit on their owners (sub-block ownership): the kernel's gather
    warps pull the foreign rows of each 128-row block over NVLink while the tensor-core warps run the blocks already
    here (`pushed`: the owners wrote them here already, the kernel only waits for their flags).
    `epilogue`: store | swiglu (c is [rows, n/2] over weights stacked [gate rows ; up rows]).
    Interface [g, g_peers, w, c, blocks, cta_epochs, ready, state, err, rows]; `ready` is row 1 of `sp.flags`."""
    out_cols = n // 2 if epilogue == "swiglu" else n
    suffix = {"store": "", "swiglu": "_swiglu"}[epilogue]
    iface = ["inout buffer<bf16>", "in buffer<u64>", "in buffer<bf16>", "out buffer<bf16>", "inout buffer<u32>",
             "inout buffer<u32>", "in buffer<u32>", "in buffer<u32>", "out buffer<i32>", "i32"]
    launches = []
    for bn, lo, hi in gemm_ranges(n, rows_max, (256, 128, 64)):
        launch = {"module": "ag_gemm", "entry": f"kern_ag_gemm_sp_bf16_tn{suffix}_n{bn}", "block": [320, 1, 1],
                  "grid": [SMS, 1, 1], "shared_mem": gemm_smem(bn),
                  "params": ["bytes<128>", "bytes<128>", "out buffer<bf16>", "i32", "i32", "i32", "i32", "out buffer<i32>",
                             "in buffer<u64>", "inout buffer<u32>", "inout buffer<u32>", "in buffer<u32>", "in buffer<u32>",
                             "i32", "i32", "i32", "i64", "i32"],
                  "args": [
                      {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
                          "param": 0, "dtype": "bf16", "dims": [k, 0], "strides": [k * 2], "box": [BK, BM], "swizzle": 128,
                          "l2_promotion": 256}}]}},
                      {"pack": {"size": 128, "fields": [{"at": 0, "tensormap": {
                          "param": 2, "dtype": "bf16", "dims": [k, n], "strides": [k * 2],
                          "box": [BK, bn // 2 if epilogue == "swiglu" else bn], "swizzle": 128, "l2_promotion": 256}}]}},
                      {"param": 3}, {"param": 9}, {"i32": n}, {"i32": k}, {"i32": out_cols}, {"param": 8}, {"param": 1},
                      {"param": 4}, {"param": 5}, {"param": 6}, {"param": 7}, {"rank": group}, {"i32": nranks},
                      {"i32": AG_MAX_BLOCKS}, {"i64": timeout_ns}, {"i32": int(pushed)}]}
        w = _when("tokens", lo, hi, rows_max)
        if w:
            launch["when"] = w
        launches.append(launch)
    return {"params": iface, "impl": {"launches": launches}}


def sp_last_rows_op(hidden: int, nranks: int, group: str = "tp", timeout_ns: int = 2_000_000_000) -> dict:
    """last[i] = the final row of sequence i, fetched from the rank that owns it. Interface
    [g_peers, last, cu_seqlens, flags, state, err, seqs]."""
    iface = ["in buffer<u64>", "out buffer<bf16>", "in buffer<i32>", "in buffer<u32>", "in buffer<u32>", "out buffer<i32>", "i32"]
    return {"params": iface, "impl": {"launches": [{
        "module": "tp_sp", "entry": "kern_sp_last_rows", "block": [256, 1, 1], "grid": ["seqs", 1, 1],
        "params": iface[:6] + ["i32", "i32", "i32", "i32", "i64"],
        "args": [{"param": i} for i in range(6)] + [{"rank": group}, {"i32": nranks}, {"param": 6}, {"i32": hidden},
                                                     {"i64": timeout_ns}]}]}}


AG_GRID = 64


def tp_allgather_op(nranks: int, slot_bytes: int, group: str = "tp", timeout_ns: int = 2_000_000_000) -> dict:
    """All-gather of one block per rank over peer memory. Interface [x, y, sym, sym_peers, flags, flag_peers, epochs, err, bytes]."""
    iface = ["in buffer<u8>", "out buffer<u8>", "inout buffer<u8>", "in buffer<u64>", "inout buffer<u32>", "in buffer<u64>",
             "inout buffer<u32>", "out buffer<i32>", "i64"]
    return {"params": iface, "impl": {"launches": [{
        "module": "tp_allreduce_norm", "entry": "kern_peer_allgather", "block": [256, 1, 1], "grid": [AG_GRID, 1, 1],
        "params": iface[:8] + ["i32", "i32", "i64", "i64", "i64", "i32"],
        "args": [{"param": i} for i in range(8)] + [{"rank": group}, {"i32": nranks}, {"param": 8}, {"i64": slot_bytes},
                                                     {"i64": timeout_ns}, {"i32": AG_GRID}]}]}}


def tp_allgather_buffers(nranks: int, slot_bytes: int, group: str = "tp") -> dict:
    return {"ag.sym": {"dtype": "u8", "shape": [2, nranks, slot_bytes], "kind": "carry", "export": True},
            "ag.sym_peers": {"dtype": "u64", "shape": [nranks], "kind": "peer", "of": "ag.sym", "group": group},
            "ag.flags": {"dtype": "u32", "shape": [nranks, AG_GRID], "kind": "carry", "export": True},
            "ag.flags_peers": {"dtype": "u64", "shape": [nranks], "kind": "peer", "of": "ag.flags", "group": group},
            "ag.epochs": {"dtype": "u32", "shape": [AG_GRID], "kind": "carry"}}


def tp_lamport_init_op(hidden: int, nranks: int) -> dict:
    """Poison the three Lamport stages (every 16-bit word 0x8000). Interface [lamport]."""
    n_words = 3 * nranks * TP_ONESHOT_ROWS * hidden // 2
    return {"params": ["out buffer<bf16>"], "impl": {"launches": [{
        "module": "misc", "entry": "kern_fill_i32", "block": [256, 1, 1], "grid": [1184, 1, 1],
        "params": ["out buffer<bf16>", "i64", "i32"], "args": [{"param": 0}, {"i64": n_words}, {"i32": -2147450880}]}]}}


def tp_buffers(hidden: int, nranks: int, rows_max: int, group: str = "tp", lamport: bool = False) -> dict:
    """Exported staging / flag buffers of the fused all-reduce and their peer address tables."""
    slot_rows = tp_slot_rows(rows_max, nranks)
    extra = {}
    if lamport:
        extra = {"tp.lamport": {"dtype": "bf16", "shape": [3, nranks, TP_ONESHOT_ROWS, hidden], "kind": "carry", "export": True},
                 "tp.lamport_peers": {"dtype": "u64", "shape": [nranks], "kind": "peer", "of": "tp.lamport", "group": group},
                 "tp.lamport_epochs": {"dtype": "u32", "shape": [TP_ONESHOT_ROWS], "kind": "carry"}}
    return {**extra,
        "tp.comm": {"dtype": "bf16", "shape": [2, nranks, slot_rows, hidden], "kind": "carry", "export": True},
        "tp.comm_peers": {"dtype": "u64", "shape": [nranks], "kind": "peer", "of": "tp.comm", "group": group},
        "tp.flags": {"dtype": "u32", "shape": [2, nranks, TP_GRID], "kind": "carry", "export": True},
        "tp.flags_peers": {"dtype": "u64", "shape": [nranks], "kind": "peer", "of": "tp.flags", "group": group},
        "tp.epochs": {"dtype": "u32", "shape": [TP_GRID], "kind": "carry"},
    }


# ---- gated DeltaNet (hybrid decoders) ----------------------------------------------------------------
def gdn_line_bytes(hk: int, hv: int, dk: int, dv: int, width: int = 4) -> tuple[int, int]:
    """(bytes of one per-sequence state line, offset of the recurrent matrix in it)."""
    conv = (width - 1) * (2 * hk * dk + hv * dv) * 2
    s_off = (conv + 255) // 256 * 256
    return s_off + hv * dv * dk * 4, s_off


def gdn_conv_op(conv_dim: int, width: int, x_stride: int, line_bytes: int, ragged: bool) -> dict:
    """Causal conv + SiLU over the first `conv_dim` channels of a row (row-parallel), then the windows kept in the
    state lines advance. Interface [x, y, state, lines, (cu_seqlens,) w, seqs, rows]."""
    assert conv_dim % 4 == 0 and x_stride % 4 == 0, "the conv kernel moves four channels (8 bytes) per thread"
    iface = ["in buffer<bf16>", "out buffer<bf16>", "inout state", "in buffer<i32>"]
    if ragged:
        iface.append("in buffer<i32>")
    iface += ["in buffer<bf16>", "i32", "i32"]
    w_at = len(iface) - 3
    if not ragged:      # one row per sequence: the conv and the window shift in one launch
        step = {"module": "gdn", "entry": "kern_gdn_conv_step_bf16", "block": [256, 1, 1], "grid": ["seqs", -(-conv_dim // 1024), 1],
                "params": ["in buffer<bf16>", "out buffer<bf16>", "inout state", "in buffer<i32>", "in buffer<bf16>", "i64", "i32",
                           "i32", "i32", "i32", "i64"],
                "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, {"param": w_at}, {"i64": 0}, {"param": w_at + 1},
                         {"i32": conv_dim}, {"i32": width}, {"i32": x_stride}, {"i64": line_bytes}]}
        return {"params": iface, "impl": {"launches": [step]}}
    cu_t, cu_a = ("in buffer<i32>", {"param": 4}) if ragged else ("i64", {"i64": 0})
    conv = {"module": "gdn", "entry": "kern_gdn_conv_bf16", "block": [256, 1, 1],
            "grid": [{"ceil_div": ["tokens", 16]} if ragged else "tokens", -(-conv_dim // 1024), 1],
            "params": ["in buffer<bf16>", "out buffer<bf16>", "in state", "in buffer<i32>", cu_t, "in buffer<bf16>", "i64",
                       "i32", "i32", "i32", "i32", "i32", "i64", "i32"],
            "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 3}, cu_a, {"param": w_at}, {"i64": 0},
                     {"param": w_at + 1}, {"param": w_at + 2}, {"i32": conv_dim}, {"i32": width}, {"i32": x_stride},
                     {"i64": line_bytes}, {"i32": 16 if ragged else 1}]}
    upd = {"module": "gdn", "entry": "kern_gdn_conv_state", "block": [256, 1, 1], "grid": ["seqs", -(-conv_dim // 256), 1],
           "params": ["in buffer<bf16>", "inout state", "in buffer<i32>", cu_t, "i32", "i32", "i32", "i32", "i64"],
           "args": [{"param": 0}, {"param": 2}, {"param": 3}, cu_a, {"i32": I32_MAX}, {"i32": conv_dim}, {"i32": width},
                    {"i32": x_stride}, {"i64": line_bytes}]}
    return {"params": iface, "impl": {"launches": [conv, upd]}}


def gdn_rule_op(hk: int, hv: int, dim: int, zba_stride: int, line_bytes: int, s_off: int, eps: float,
                ragged: bool, chunked: bool = True) -> dict:
    """Gated delta rule (value rows split over CTAs) + gated RMSNorm.
    Interface [qkv, zba, out, state, lines, A_log, dt_bias, norm_w] for one row per sequence (the fused step), or
    [qkv, zba, out, state, lines, cu_seqlens, A_log, dt_bias, norm_w, seqs] for ragged rows; `zba` points at the z|b|a
    columns of the projection's row. Ragged rows of 128-wide heads take the chunked (WY) pair of launches."""
    iface = ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "inout state", "in buffer<i32>"]
    if not ragged:
        # one row per sequence: the fused step (state by bulk copy, rule, gated norm) in one launch
        iface += ["in buffer<f32>", "in buffer<f32>", "in buffer<bf16>"]
        step = {"module": "gdn", "entry": f"kern_gdn_step_k{dim}_v{dim}", "block": [256, 1, 1], "grid": [hv, "seqs", 1],
                "shared_mem": dim * dim * 4 + (4 * dim + 16) * 4 + 16,
                "params": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "inout state", "in buffer<i32>",
                           "in buffer<f32>", "in buffer<f32>", "in buffer<bf16>"] + ["i32"] * 7 + ["i64", "i64", "f32"],
                "args": [{"param": i} for i in range(8)] + [
                    {"i32": I32_MAX}, {"i32": hk}, {"i32": hv}, {"i32": zba_stride}, {"i32": 0}, {"i32": hv * dim},
                    {"i32": hv * dim + hv}, {"i64": line_bytes}, {"i64": s_off}, {"f32": eps}]}
        return {"params": iface, "impl": {"launches": [step]}}
    iface.append("in buffer<i32>")
    at = len(iface)
    tb = 32 if ragged else 1          # tokens staged per pass
    iface += ["in buffer<f32>", "in buffer<f32>", "in buffer<bf16>", "i32"]      # ..., A_log, dt_bias, norm_w, seqs
    lp = ["in buffer<bf16>", "in buffer<bf16>", "out buffer<f32>", "inout state", "in buffer<i32>",
          "in buffer<i32>" if ragged else "i64", "in buffer<f32>", "in buffer<f32>"] + ["i32"] * 6 + ["i64", "i64", "i32"]
    args = [{"param": 0}, {"param": 1}, {"scratch": "o_raw"}, {"param": 3}, {"param": 4},
            {"param": 5} if ragged else {"i64": 0}, {"param": at}, {"param": at + 1}, {"param": at + 3}, {"i32": hk},
            {"i32": hv}, {"i32": zba_stride}, {"i32": hv * dim}, {"i32": hv * dim + hv}, {"i64": line_bytes}, {"i64": s_off},
            {"i32": tb}]
    norm = {"module": "gdn", "entry": "kern_gdn_gate_norm_bf16", "block": [128, 1, 1], "grid": [-(-hv // 4), "tokens", 1],
            "params": ["in buffer<f32>", "in buffer<bf16>", "out buffer<bf16>", "in buffer<bf16>", "i32", "i32", "i32", "i32",
                       "i32", "f32"],
            "args": [{"scratch": "o_raw"}, {"param": 1}, {"param": 2}, {"param": at + 2}, {"i32": I32_MAX}, {"i32": hv},
                     {"i32": dim}, {"i32": zba_stride}, {"i32": 0}, {"f32": eps}]}
    if chunked and dim == 128:
        # prefill rows in the chunked (WY) form: factors per (64-token chunk, head) on the tensor cores, then one pass
        # over the chunks with the state on chip
        names = ["gw", "gq", "gk", "gu", "gm", "gc"]
        sc = [{"scratch": n} for n in names]
        prep = {"module": "gdn_chunk", "entry": "kern_gdn_chunk_prep_k128_v128", "block": [256, 1, 1],
                "grid": [{"add": [{"ceil_div": ["tokens", 64]}, "seqs"]}, hv, 1],
                "shared_mem": (2 * 64 * 132 + 64 * 68 + 2 * 64) * 4,
                "params": ["in buffer<bf16>", "in buffer<bf16>", "in buffer<i32>", "in buffer<f32>", "in buffer<f32>"] +
                          ["out buffer<f32>"] * 6 + ["i32"] * 6,
                "args": [{"param": 0}, {"param": 1}, {"param": 5}, {"param": at}, {"param": at + 1}, *sc,
                         {"param": at + 3}, {"i32": hk}, {"i32": hv}, {"i32": zba_stride}, {"i32": hv * dim},
                         {"i32": hv * dim + hv}]}
        walk = {"module": "gdn_chunk", "entry": "kern_gdn_chunk_rule_k128_v128", "block": [256, 1, 1],
                "grid": [hv * 2, "seqs", 1], "shared_mem": (64 * 132 * 3 + 64 * 136 + 64 * 68 + 2 * 64 * 72) * 4,
                "params": ["in buffer<f32>"] * 6 + ["out buffer<f32>", "inout state", "in buffer<i32>", "in buffer<i32>",
                                                    "i32", "i32", "i64", "i64"],
                "args": [*sc, {"scratch": "o_raw"}, {"param": 3}, {"param": 4}, {"param": 5}, {"param": at + 3}, {"i32": hv},
                         {"i64": line_bytes}, {"i64": s_off}]}
        scratch = {n: {"dtype": "f32", "shape": ["tokens", hv * 128]} for n in names[:4]}
        scratch["gm"] = {"dtype": "f32", "shape": ["tokens", hv * 64]}
        scratch["gc"] = {"dtype": "f32", "shape": ["tokens", hv]}
        scratch["o_raw"] = {"dtype": "f32", "shape": ["tokens", hv * dim]}
        return {"params": iface, "impl": {"launches": [prep, walk, norm], "scratch": scratch}}
    rows_cta = 16          # value rows per CTA
    rule = {"module": "gdn", "entry": f"kern_gdn_rule_{'' if ragged else 'dec_'}k{dim}_v{dim}", "block": [256, 1, 1],
            "grid": [hv * (dim // rows_cta), "seqs", 1], "shared_mem": tb * (2 * dim + rows_cta + 4) * 4, "params": lp,
            "args": args}
    return {"params": iface, "impl": {"launches": [rule, norm],
                                      "scratch": {"o_raw": {"dtype": "f32", "shape": ["tokens", hv * dim]}}}}


def sigmoid_mul_op(d: int, x_stride: int, gate_stride: int) -> dict:
    """out[t, :d] = x[t, :d] * sigmoid(gate[t, :d]). Interface [x, gate, out]."""
    return {"params": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>"], "impl": {"launches": [{
        "module": "norm_embed", "entry": "kern_sigmoid_mul_bf16", "block": [256, 1, 1],
        "grid": ["tokens", max(1, -(-d // 256)), 1],
        "params": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "i32", "i32", "i32", "i32"],
        "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"i32": I32_MAX}, {"i32": d}, {"i32": x_stride},
                 {"i32": gate_stride}]}]}}


# ---- per-key-decay delta rule (Kimi Delta Attention) and latent attention ---------------------------------------
def kda_rule_op(hk: int, hv: int, dim: int, zba_stride: int, line_bytes: int, s_off: int, eps: float, ragged: bool,
                chunked: bool = True) -> dict:
    """Delta rule with a decay per key channel + gated RMSNorm. `zba` points at the z|b columns of the projection's
    row and `gk` at its hv * dim gate columns (same row stride).
    Interface [qkv, zba, gk, out, state, lines, A_log, dt_bias, norm_w] for one row per sequence (the fused step), or
    [qkv, zba, gk, out, state, lines, cu_seqlens, A_log, dt_bias, norm_w, seqs] for ragged rows (heads of 128 in the
    chunked form, others token by token)."""
    assert dim in (64, 128)
    iface = ["in buffer<bf16>", "in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "inout state", "in buffer<i32>"]
    if not ragged:
        iface += ["in buffer<f32>", "in buffer<f32>", "in buffer<bf16>"]
        step = {"module": "gdn", "entry": f"kern_kda_step_k{dim}_v{dim}", "block": [256, 1, 1], "grid": [hv, "seqs", 1],
                "shared_mem": dim * dim * 4 + (4 * dim + 16) * 4 + 16 + dim * 4,
                "params": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>", "inout state", "in buffer<i32>",
                           "in buffer<f32>", "in buffer<f32>", "in buffer<bf16>", "in buffer<bf16>"] + ["i32"] * 7 +
                          ["i64", "i64", "f32"],
                "args": [{"param": 0}, {"param": 1}, {"param": 3}, {"param": 4}, {"param": 5}, {"param": 6}, {"param": 7},
                         {"param": 8}, {"param": 2}, {"i32": I32_MAX}, {"i32": hk}, {"i32": hv}, {"i32": zba_stride}, {"i32": 0},
                         {"i32": hv * dim}, {"i32": zba_stride}, {"i64": line_bytes}, {"i64": s_off}, {"f32": eps}]}
        return {"params": iface, "impl": {"launches": [step]}}
    iface += ["in buffer<i32>", "in buffer<f32>", "in buffer<f32>", "in buffer<bf16>", "i32"]
    tb = 32
    rule = {"module": "gdn", "entry": f"kern_kda_rule_k{dim}_v{dim}", "block": [256, 1, 1], "grid": [hv * (dim // 16), "seqs", 1],
            "shared_mem": tb * (3 * dim + 16 + 4) * 4,
            "params": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<f32>", "inout state", "in buffer<i32>", "in buffer<i32>",
                       "in buffer<f32>", "in buffer<f32>", "in buffer<bf16>"] + ["i32"] * 6 + ["i64", "i64", "i32"],
            "args": [{"param": 0}, {"param": 1}, {"scratch": "o_raw"}, {"param": 4}, {"param": 5}, {"param": 6}, {"param": 7},
                     {"param": 8}, {"param": 2}, {"param": 10}, {"i32": hk}, {"i32": hv}, {"i32": zba_stride}, {"i32": hv * dim},
                     {"i32": zba_stride}, {"i64": line_bytes}, {"i64": s_off}, {"i32": tb}]}
    norm = {"module": "gdn", "entry": "kern_gdn_gate_norm_bf16", "block": [128, 1, 1], "grid": [-(-hv // 4), "tokens", 1],
            "params": ["in buffer<f32>", "in buffer<bf16>", "out buffer<bf16>", "in buffer<bf16>", "i32", "i32", "i32", "i32",
                       "i32", "f32"],
            "args": [{"scratch": "o_raw"}, {"param": 1}, {"param": 3}, {"param": 9}, {"i32": I32_MAX}, {"i32": hv},
                     {"i32": dim}, {"i32": zba_stride}, {"i32": 0}, {"f32": eps}]}
    if chunked and dim == 128:
        # prefill rows in the chunked (WY) form: pairwise sums with a weight per key on the CUDA cores, the solve and the
        # products with the state on the tensor cores, one pass over the chunks with the state on chip
        names = ["gw", "gq", "gk", "gu", "gm", "gd"]
        sc = [{"scratch": n} for n in names]
        prep = {"module": "gdn_chunk", "entry": "kern_kda_chunk_prep_k128_v128", "block": [256, 1, 1],
                "grid": [{"add": [{"ceil_div": ["tokens", 64]}, "seqs"]}, hv, 1],
                "shared_mem": (3 * 64 * 132 + 64 + 3 * 128) * 4,
                "params": ["in buffer<bf16>", "in buffer<bf16>", "in buffer<bf16>", "in buffer<i32>", "in buffer<f32>",
                           "in buffer<f32>"] + ["out buffer<f32>"] * 6 + ["i32"] * 6,
                "args": [{"param": 0}, {"param": 1}, {"param": 2}, {"param": 6}, {"param": 7}, {"param": 8}, *sc,
                         {"param": 10}, {"i32": hk}, {"i32": hv}, {"i32": zba_stride}, {"i32": hv * dim}, {"i32": zba_stride}]}
        walk = {"module": "gdn_chunk", "entry": "kern_kda_chunk_rule_k128_v128", "block": [256, 1, 1],
                "grid": [hv * 2, "seqs", 1], "shared_mem": (64 * 132 * 3 + 64 * 136 + 64 * 68 + 2 * 64 * 72) * 4,
                "params": ["in buffer<f32>"] * 6 + ["out buffer<f32>", "inout state", "in buffer<i32>", "in buffer<i32>",
                                                    "i32", "i32", "i64", "i64"],
                "args": [*sc, {"scratch": "o_raw"}, {"param": 4}, {"param": 5}, {"param": 6}, {"param": 10}, {"i32": hv},
                         {"i64": line_bytes}, {"i64": s_off}]}
        scratch = {n: {"dtype": "f32", "shape": ["tokens", hv * 128]} for n in names}
        scratch["gm"] = {"dtype": "f32", "shape": ["tokens", hv * 64]}
        scratch["o_raw"] = {"dtype": "f32", "shape": ["tokens", hv * dim]}
        return {"params": iface, "impl": {"launches": [prep, walk, norm], "scratch": scratch}}
    return {"params": iface, "impl": {"launches": [rule, norm],
                                      "scratch": {"o_raw": {"dtype": "f32", "shape": ["tokens", hv * dim]}}}}


MLA_DQK, MLA_DV = 576, 512
MLA_SMEM = 1024 + 2 * 64 * MLA_DQK * 2 + 16 * (MLA_DQK + 8) * 2 + 16 * (64 + 8) * 2 + 2 * 8 * 16 * 4 + 128


def mla_rope_append_op(heads: int, lat_stride: int, eps: float, max_pos: int) -> dict:
    """Latent row of a token (RMS-normed 512 compressed columns + rotated 64 positional ones) into the paged latent
    cache, and the rotation of the positional 64 columns of every head's query, in place.
    Interface [latent columns of the projection's row, q, latent state, positions, slots, cos, sin, norm weight, err]."""
    iface = ["in buffer<bf16>", "inout buffer<bf16>", "inout state", "in buffer<i64>", "in buffer<i64>", "in buffer<f32>",
             "in buffer<f32>", "in buffer<bf16>", "out buffer<i32>"]
    return {"params": iface, "impl": {"launches": [{
        "module": "mla_decode", "entry": "kern_mla_rope_append_bf16", "block": [128, 1, 1], "grid": ["tokens", 1, 1],
        "params": iface[:8] + ["i32", "i32", "i32", "i32", "f32", "i64", "i32", "out buffer<i32>"],
        "args": [{"param": i} for i in range(8)] + [{"i32": I32_MAX}, {"i32": heads}, {"i32": lat_stride},
                                                     {"i32": heads * MLA_DQK}, {"f32": eps}, {"i64": I64_MAX}, {"i32": max_pos},
                                                     {"param": 8}]}]}}


def mla_rows_op() -> dict:
    """One attention row per token of a ragged call. Interface [positions, cu_seqlens, row_seq, row_len, seqs, tokens]."""
    iface = ["in buffer<i64>", "in buffer<i32>", "out buffer<i32>", "out buffer<i32>", "i32", "i32"]
    return {"params": iface, "impl": {"launches": [{
        "module": "mla_decode", "entry": "kern_mla_rows", "block": [128, 1, 1], "grid": [{"ceil_div": ["tokens", 128]}, 1, 1],
        "params": ["in buffer<i64>", "in buffer<i32>", "i32", "i32", "out buffer<i32>", "out buffer<i32>"],
        "args": [{"param": 0}, {"param": 1}, {"param": 4}, {"param": 5}, {"param": 2}, {"param": 3}]}]}}


def mla_attn_op(heads: int, page_size: int, table_width: int, ragged: bool, head_width: int = 192, seqs_max: int = 0,
                sms: int = SMS) -> dict:
    """Absorbed latent attention: every head attends over the shared 576-wide latent rows, values their first 512
    columns. One row per sequence: interface [q, latent state, out, block_table, seq_lens, err], the context split over
    CTAs by `when` ranges of the batch (partials merged by a second launch) so that a few long sequences still fill
    the machine; ragged rows bring [.., row_len, err, row_seq] — a row reads its sequence's table row and attends over
    its own causal reach."""
    assert page_size % 64 == 0 or 64 % page_size == 0
    iface = ["in buffer<bf16>", "in state", "out buffer<bf16>", "in buffer<i32>", "in buffer<i32>", "out buffer<i32>"]
    if ragged:
        iface.append("in buffer<i32>")
    blocks = -(-heads // 16)
    ranges, hi = [], seqs_max
    if ragged or not seqs_max:
        ranges = [(1, 1, seqs_max)]
    else:
        for splits in (1, 2, 4, 8, 16, 32):
            lo = 1 if splits == 32 else max(1, -(-sms // (blocks * splits)))
            if lo <= hi:
                ranges.append((splits, lo, hi))
                hi = lo - 1
            if hi < 1:
                break
    max_splits = max(s for s, _, _ in ranges)
    launches = []
    for splits, lo, hi in ranges:
        when = {"var": "seqs"}
        if lo > 1:
            when["min"] = lo
        if seqs_max and hi < seqs_max:
            when["max"] = hi
        part = splits > 1
        lp = ["bytes<128>", "in buffer<bf16>", "out buffer<bf16>", "out buffer<f32>" if part else "i64",
              "out buffer<f32>" if part else "i64", "in buffer<i32>", "in buffer<i32>"] + ["i32"] * 8 + \
             ["f32", "out buffer<i32>", "in buffer<i32>" if ragged else "i64"]
        ws = [{"scratch": "ws_o"}, {"scratch": "ws_ml"}] if part else [{"i64": 0}, {"i64": 0}]
        args = [_kv_map(MLA_DQK, page_size, 1), {"param": 0}, {"param": 2}, *ws, {"param": 3}, {"param": 4},
                {"i32": I32_MAX}, {"i32": heads}, {"i32": heads * MLA_DQK}, {"i32": heads * MLA_DV}, {"i32": table_width},
                {"i32": page_size}, {"i32": splits}, {"i32": I32_MAX}, {"f32": (head_width ** -0.5) * 1.4426950408889634},
                {"param": 5}, {"param": 6} if ragged else {"i64": 0}]
        launch = {"module": "mla_decode", "entry": "kern_mla_decode_bf16", "block": [288, 1, 1],
                  "grid": [blocks, "tokens" if ragged else "seqs", splits], "shared_mem": MLA_SMEM, "params": lp, "args": args}
        merge = {"module": "attn_paged", "entry": "kern_attn_merge_splits", "block": [256, 1, 1],
                 "grid": [{"mul": ["tokens", heads]}, 1, 1],
                 "params": ["in buffer<f32>", "in buffer<f32>", "out buffer<bf16>", "i32", "i32", "i32", "i32", "i32"],
                 "args": [{"scratch": "ws_o"}, {"scratch": "ws_ml"}, {"param": 2}, {"i32": I32_MAX}, {"i32": heads},
                          {"i32": MLA_DV}, {"i32": splits}, {"i32": heads * MLA_DV}]}
        for l in ([launch, merge] if part else [launch]):
            if len(when) > 1:
                l["when"] = when
            launches.append(l)
    impl = {"launches": launches}
    if max_splits > 1:
        impl["scratch"] = {"ws_o": {"dtype": "f32", "shape": ["tokens", heads * max_splits * MLA_DV]},
                           "ws_ml": {"dtype": "f32", "shape": ["tokens", heads * max_splits * 2]}}
    return {"params": iface, "impl": impl}
