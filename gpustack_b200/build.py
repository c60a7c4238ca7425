"""Build libb200.so (the sm_100a kernel library) in-tree with nvcc.

The shared object lands next to the sources (gpustack_b200/csrc/libb200.so) so that it travels
with the repository snapshot to the GPU box; it is git-ignored.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIB = CSRC / "libb200.so"
SOURCES = [
    "runtime.cu",
    "norm.cu",
    "rope_kv.cu",
    "elementwise.cu",
    "gemm_tcgen05.cu",
    "quant_fp8.cu",
    "moe.cu",
    "attention.cu",
    "attention_prefill_tc.cu",
    "allreduce.cu",
    "gemm_simt.cu",
    "postnorm.cu",
    "attention_sink.cu",
    "mlstm.cu",
    "streams.cu",
    "latent.cu",
    "latent_attention_mma.cu",
    "gemm_simt_grouped.cu",
    "moe_biased.cu",
    "prenorm.cu",
    "rot_prep.cu",
    "linear_attn.cu",
    "sandwich.cu",
    "gated_recurrence.cu",
    "gated_linear_attn.cu",
]
# What a layer-list decoder (attention with a softmax sink / matrix-memory recurrence, norm after the
# sum) launches: a fresh checkout that only serves such a model compiles these and nothing else.
LAYER_LIST_SOURCES = [
    "runtime.cu",
    "elementwise.cu",
    "gemm_tcgen05.cu",
    "gemm_simt.cu",
    "postnorm.cu",
    "attention_sink.cu",
    "mlstm.cu",
]
# ... plus the tensor-core attention kernels when some attention layer has tile-sized heads
ATTENTION_TC_SOURCES = ["attention.cu", "attention_prefill_tc.cu"]
# What a pre-norm decoder over residual streams with latent attention and gated / routed feed-forwards launches
STREAMS_LATENT_SOURCES = [
    "runtime.cu",
    "elementwise.cu",
    "gemm_tcgen05.cu",
    "gemm_simt.cu",
    "gemm_simt_grouped.cu",
    "streams.cu",
    "latent.cu",
    "latent_attention_mma.cu",
    "attention_sink.cu",
]
ROUTED_SOURCES = ["moe.cu", "moe_biased.cu"]
# What a pre-norm decoder with one norm per layer (mixer and feed-forward side by side), rotary attention in a
# sliding window and decayed linear attention launches; routed feed-forwards add ROUTED_SOURCES
PARALLEL_SOURCES = [
    "runtime.cu",
    "elementwise.cu",
    "gemm_tcgen05.cu",
    "gemm_simt.cu",
    "gemm_simt_grouped.cu",
    "streams.cu",
    "prenorm.cu",
    "rot_prep.cu",
    "attention_sink.cu",
    "linear_attn.cu",
]


# What a decoder with a norm before and after every sublayer, input convolutions, rotary attention (also with pooled
# blocks beside a window), gated diagonal recurrences and gated linear attention launches
SANDWICH_SOURCES = [
    "runtime.cu",
    "elementwise.cu",
    "gemm_tcgen05.cu",
    "gemm_simt.cu",
    "gemm_simt_grouped.cu",
    "sandwich.cu",
    "rot_prep.cu",
    "attention_sink.cu",
    "linear_attn.cu",
    "gated_recurrence.cu",
    "gated_linear_attn.cu",
]


def layer_list_sources(mcfg):
    """(tag, sources) of the library a process serving this layer-list model needs."""
    if getattr(mcfg, "residual", "post_ln") == "sandwich":
        attn = [l.mixer if l.mixer.kind == "attention" else l.mixer.left for l in mcfg.layers
                if l.mixer.kind in ("attention", "side_by_side")]
        tc = any(a.tokens_tile_sized for a in attn)       # a window's tokens too, when pooled blocks follow
        return ("sandwich_tc", SANDWICH_SOURCES + ATTENTION_TC_SOURCES) if tc else ("sandwich", list(SANDWICH_SOURCES))
    if getattr(mcfg, "residual", "post_ln") == "parallel":
        routed = any(l.mlp is not None and l.mlp.kind == "moe" for l in mcfg.layers)
        tc = any(l.mixer.kind == "attention" and l.mixer.tile_sized for l in mcfg.layers)
        tag = "parallel" + ("_routed" if routed else "") + ("_tc" if tc else "")
        return tag, PARALLEL_SOURCES + (ROUTED_SOURCES if routed else []) + (ATTENTION_TC_SOURCES if tc else [])
    if getattr(mcfg, "residual", "post_ln") == "streams":
        routed = any(l.mlp is not None and l.mlp.kind == "moe" for l in mcfg.layers)
        return ("streams_routed", STREAMS_LATENT_SOURCES + ROUTED_SOURCES) if routed else ("streams", list(STREAMS_LATENT_SOURCES))
    tc = any(l.mixer.kind == "attention" and l.mixer.tile_sized for l in mcfg.layers)
    return ("layer_list_tc", LAYER_LIST_SOURCES + ATTENTION_TC_SOURCES) if tc else ("layer_list", list(LAYER_LIST_SOURCES))


NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _file_digest(src: Path, headers) -> str:
    h = hashlib.sha256()
    for p in [src, *headers]:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def subset_lib(tag: str) -> Path:
    return CSRC / f"libb200_{tag}.so"


def build(force: bool = False, verbose: bool = False, variant: str = "", sources=None, tag: str = "") -> Path:
    """variant "" = the product library (dependents released after the kernel's own dependency wait);
    "early" = libb200_early.so, the experimental build with the entry-time trigger
    (-DB200_PDL_EARLY_TRIGGER), kept only to reproduce the hazard documented beside pdl_wait().
    sources + tag: link only those files into libb200_<tag>.so (same ABI, fewer symbols) -- what a
    process that serves one model family needs on a fresh checkout.  Objects are cached per source
    file, so a later full build compiles only what is still missing."""
    names = list(SOURCES if sources is None else sources)
    srcs = [CSRC / s for s in names]
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [CSRC.parent.parent / "include" / "b200.h"]
    if sources is not None and not tag:
        raise ValueError("a subset build needs a tag")
    lib = (LIB if not tag else subset_lib(tag)) if not variant else CSRC / f"libb200_{variant}.so"
    extra = {"": [], "early": ["-DB200_PDL_EARLY_TRIGGER=1"]}[variant]
    objdir = CSRC / ("build" if not variant else f"build_{variant}")
    stamp = objdir / (f"stamp_{tag}" if tag else "stamp")
    digests = {src: _file_digest(src, headers) + variant for src in srcs}
    digest = hashlib.sha256("".join(f"{s.name}:{d};" for s, d in sorted(digests.items())).encode()).hexdigest()
    if not force and lib.exists() and stamp.exists() and stamp.read_text() == digest:
        return lib
    nvcc = _nvcc()
    objdir.mkdir(exist_ok=True)

    def compile_one(src: Path):
        obj = objdir / (src.stem + ".o")
        mark = objdir / (src.stem + ".digest")
        if not force and obj.exists() and mark.exists() and mark.read_text() == digests[src]:
            return obj
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = objdir / (src.stem + ".log")
        log.write_text(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        mark.write_text(digests[src])
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = lib.with_suffix(f".{os.getpid()}.tmp")
    cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    stamp.write_text(digest)
    return lib


def is_current(lib: Path = LIB) -> bool:
    """True when `lib` (the full library by default) exists and was built from the sources as they are."""
    if lib != LIB or not lib.exists():
        return False
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [CSRC.parent.parent / "include" / "b200.h"]
    stamp = CSRC / "build" / "stamp"
    digests = {CSRC / s: _file_digest(CSRC / s, headers) for s in SOURCES}
    digest = hashlib.sha256("".join(f"{s.name}:{d};" for s, d in sorted(digests.items())).encode()).hexdigest()
    return stamp.exists() and stamp.read_text() == digest


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, variant="early" if "--early" in sys.argv else ""))
