"""The engine's kernels as Python calls over torch tensors (ctypes into the built libraries).

There is no fallback: if a library cannot be built or loaded, or a kernel
refuses a size, the call raises. Calls launch on torch's current stream.
"""
from __future__ import annotations

import bisect
import ctypes
import os
from typing import Dict, Optional

import numpy as np
import torch

from . import build

_DT = {torch.float32: 0, torch.bfloat16: 1}

_ERRORS = {
    -1: "unsupported dtype",
    -2: "a size the kernel refuses",
    -3: "a pointer or stride is not aligned as the kernel needs",
    -4: "a size beyond the kernel's stated maximum",
}


class KernelError(RuntimeError):
    pass


def _check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[rc]}")
    if rc < 0:
        raise KernelError(f"{what}: library error {rc}")
    raise KernelError(f"{what}: CUDA error {rc} at launch")


def _p(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class _PinnedStream:
    """While active, the kernels launch on the given stream handle without asking torch for the current stream at
    every launch (that question costs several microseconds, a hundred times a step)."""

    def __init__(self, kernels, handle):
        self.kernels, self.handle, self.before = kernels, handle, None

    def __enter__(self):
        self.before = self.kernels._stream_handle
        self.kernels._stream_handle = ctypes.c_void_p(self.handle) if self.handle is not None else None
        return self

    def __exit__(self, *exc):
        self.kernels._stream_handle = self.before
        return False


def core_jobs():
    return [
        {"name": "sb_core", "sources": ["elementwise.cu", "skinny_linear.cu", "gemm_tcgen05.cu"]},
        {"name": "sb_gemm", "sources": ["gemm_cublas.cu"], "libs": ["cublas"]},
    ]


def attention_job(head_dim: int):
    return {"name": f"sb_attention_hd{head_dim}", "sources": ["attention_simt.cu", "attention_mma.cu", "attention_tc.cu"],
            "defines": [f"SB_HEAD_DIM={head_dim}"]}


def layer_run_job(head_dim: int):
    # SERVE_B200_STACK_DEFINES: extra -D settings for experiments with the kernel's constants (space separated)
    extra = os.environ.get("SERVE_B200_STACK_DEFINES", "").split()
    return {"name": f"sb_stack_hd{head_dim}", "sources": ["decode_stack.cu"], "defines": [f"SB_HEAD_DIM={head_dim}"] + extra}


SUPPORTED_HEAD_DIMS = tuple(range(16, 257, 16))
# head sizes for which the kernel that runs whole layers of a decoding step is built
LAYER_RUN_HEAD_DIMS = (64, 128)

# one layer as decode_stack.h lays it out (SbStackLayer)
_STACK_LAYER = np.dtype([("wqkv", "u8"), ("wo", "u8"), ("wgu", "u8"), ("wdown", "u8"), ("norm1", "u8"), ("norm2", "u8"),
                         ("inv_freq", "u8"), ("kc", "u8"), ("vc", "u8"), ("eps1", "f4"), ("eps2", "f4"), ("scale_log2", "f4"),
                         ("rot", "i4"), ("window", "i4"), ("norm_f32", "i4"), ("group", "i4"), ("num_pages", "i4"),
                         ("write_cache", "i4"), ("pad", "i4")])
_STACK_MAX_GROUPS = 4
_STACK_MAX_ROWS = 16


class LayerRunPlan:
    """A run of layers that one launch of the decode-stack kernel takes: the layers' table on the device and what
    every step needs to call the kernel."""

    def __init__(self, lib, table, keep, n_layers, hidden, heads, kv_heads, head_dim, inter, groups, page_size, blocks):
        self.lib, self.table, self.keep, self.n_layers = lib, table, keep, n_layers
        self.hidden, self.heads, self.kv_heads, self.head_dim, self.inter = hidden, heads, kv_heads, head_dim, inter
        self.groups, self.page_size, self.blocks = groups, page_size, blocks
        self.takes: Dict[int, bool] = {}


def all_jobs():
    """Every library the engine can ask for (the build check compiles them all)."""
    return core_jobs() + [attention_job(d) for d in SUPPORTED_HEAD_DIMS] + [layer_run_job(d) for d in LAYER_RUN_HEAD_DIMS]


class CudaKernels:
    """Loads (building if needed) the libraries and exposes one method per kernel."""

    def __init__(self, device="cuda:0", head_dims=(), verbose: bool = True):
        self.device = torch.device(device)
        if self.device.type == "cuda" and torch.cuda.is_available():
            self.TARGET_BLOCKS = torch.cuda.get_device_properties(self.device).multi_processor_count
        jobs = core_jobs() + [attention_job(d) for d in sorted(set(head_dims))]
        for j in jobs:
            j["verbose"] = verbose
        paths = build.build_many(jobs)
        self.paths = dict(paths)
        self._core = ctypes.CDLL(paths["sb_core"])
        self._gemm = ctypes.CDLL(paths["sb_gemm"])
        self._attn: Dict[int, ctypes.CDLL] = {}
        for d in set(head_dims):
            self._attn[d] = ctypes.CDLL(paths[f"sb_attention_hd{d}"])
            self._attn[d].sb_attention_mma_scratch_bytes.restype = ctypes.c_longlong
        self._verbose = verbose
        self._errors: Optional[torch.Tensor] = None
        self.force_simt_attention = False   # tests: run bfloat16 through the plain-arithmetic kernel
        self.use_skinny_linear = True       # tests: False sends every product to the library
        self.use_tcgen05 = True             # tests: False keeps many-row products in the library
        self.fuse_rope = True               # tests: False runs the rotary kernel after the q/k/v product
        self.use_tcgen05_attention = True   # tests: False keeps prompt portions on the mma.sync kernel
        if os.environ.get("SERVE_B200_TCGEN05_PLAIN") == "1":     # measurements: plain products on the tiles too
            self.tcgen05_for_plain_products = True
        self._stream_handle = None           # set by on_current_stream(): the stream every launch goes to
        self._routes: Dict[tuple, int] = {}  # which product kernel takes a shape (asked of the libraries once)
        self._tc_attention_ok: Dict[tuple, bool] = {}
        self._split_scratch = None           # partial results of the split-key merge
        self._sample_work = None
        self._keep = []
        self._tickets = []                   # zeroed int32 buffers of the split-key merge (kept alive for graphs)
        self.launches = 0         # launches of this engine's own kernels
        self.library_calls = 0    # library matrix products
        # Small decoding steps can run all layers in ONE launch (csrc/decode_stack.cu). Measured on a B200 at the
        # Llama-3.2-1B shape it is slower than the chain of separate kernels (about 80 us a layer against 42), so it is
        # off unless asked for (tests, and SERVE_B200_LAYER_RUNS=1 for measurements).
        self.use_layer_runs = os.environ.get("SERVE_B200_LAYER_RUNS", "0") == "1"
        self._stack: Dict[int, ctypes.CDLL] = {}
        self._stack_sync = None              # two counters of the layer-run kernel's grid barrier (zero between launches)
        self._stack_partials = None
        self.layer_runs = 0                  # launches of the layer-run kernel
        self.layer_run_timing = None         # profiles: an int64 tensor [layers * 10] that receives block 0's phase stamps

    # ---- stream -----------------------------------------------------------
    def on_current_stream(self):
        """Context manager: look torch's current stream up once and launch on it until the block ends.
        Enter it again after switching streams (graph capture does)."""
        return _PinnedStream(self, torch.cuda.current_stream(self.device).cuda_stream)

    def _s(self):
        h = self._stream_handle
        return h if h is not None else ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    # ---- checks -----------------------------------------------------------
    @staticmethod
    def check_attention_shape(heads: int, kv_heads: int, head_dim: int) -> None:
        if head_dim % 16 or not (16 <= head_dim <= 256):
            raise KernelError(f"head_dim {head_dim} is not supported: the attention kernels take multiples of 16 from 16 to 256")
        if heads % kv_heads:
            raise KernelError(f"heads {heads} is not a multiple of kv_heads {kv_heads}")
        if heads > 65535:
            raise KernelError("more than 65535 heads")

    def _attention_lib(self, head_dim: int):
        lib = self._attn.get(head_dim)
        if lib is None:
            self.check_attention_shape(1, 1, head_dim)
            job = attention_job(head_dim)
            job["verbose"] = self._verbose
            path = build.build_library(**job)
            self.paths[job["name"]] = path
            lib = self._attn[head_dim] = ctypes.CDLL(path)
            lib.sb_attention_mma_scratch_bytes.restype = ctypes.c_longlong
        return lib

    def errors_tensor(self) -> torch.Tensor:
        if self._errors is None:
            # [0]: cache writes that met a missing page; [1]: a bounded wait inside a kernel ran out
            self._errors = torch.zeros(4, dtype=torch.int32, device=self.device)
        return self._errors

    # The tensor-memory product works in 128 x 256 tiles, one CTA per SM: with fewer tiles than this most SMs
    # would idle and the library's split-k kernels are the better choice.
    TCGEN05_MIN_TILES = 96
    # A product without an epilogue of its own (output and down projection) goes to the library at every row count above the
    # few-rows kernel's: measured on a B200 at the 1B shapes from 128 to 4,096 rows the library is the faster one (2,048
    # rows: 14.9 against 16.2 us and 47.5 against 52.3 us; 3,072 rows: 20.7 / 26.9 and 69.7 / 95.9), and a prompt step of
    # 2,048 / 4,096 / 8,192 tokens went from 4.48 / 8.94 / 23.3 to 4.31 / 8.46 / 20.9 ms. The tiles earn their place where
    # an epilogue is fused (gate/up + SwiGLU, q/k/v + rotation + cache write). True: plain products use the tiles too (tests).
    tcgen05_for_plain_products = False

    def _tcgen05_worthwhile(self, m: int, n_acc: int) -> bool:
        return self.use_tcgen05 and (-(-m // 128)) * (-(-n_acc // 256)) >= self.TCGEN05_MIN_TILES

    def _wait_flag(self):
        return ctypes.c_void_p(self.errors_tensor().data_ptr() + 4)

    def check_errors(self) -> None:
        """Raise if a kernel met a page id or block index outside its table (synchronises)."""
        if self._errors is not None:
            n, timeouts = self._errors[:2].tolist()
            if n or timeouts:
                self._errors.zero_()
                if self._stack_sync is not None:
                    self._stack_sync.zero_()     # a barrier that gave up leaves its counters as they were
                if timeouts:
                    raise KernelError("a wait on a copy or tensor-core barrier inside a kernel ran out; the step's results are not valid")
                raise KernelError(f"{n} cache writes met a missing page or a block index beyond the block table")

    # ---- kernels ----------------------------------------------------------
    def fetch_ints(self, host_pinned, dev, n: int) -> None:
        """dev[:n] = host_pinned[:n] (int32, n a multiple of 4), copied by a kernel that reads the pinned host buffer."""
        self.launches += 1
        _check(self._core.sb_fetch_ints(_p(host_pinned), _p(dev), n, self._s()), "fetch of the step's inputs")

    def embedding(self, tokens, table, out, last_token=None) -> None:
        """out[t] = table[tokens[t]]; an id -(s+1) is replaced by last_token[s] (the token last sampled for slot s)."""
        self.launches += 1
        _check(self._core.sb_embedding(_p(tokens), _p(table), _p(out), tokens.shape[0], table.shape[1], table.shape[0],
                                       _DT[table.dtype], _p(last_token), last_token.shape[0] if last_token is not None else 0,
                                       self._s()), "embedding")

    def add_rmsnorm(self, x, delta, weight, eps, out) -> None:
        self.launches += 1
        _check(self._core.sb_add_rmsnorm(_p(x), _p(delta), _p(None), _p(weight), _DT[weight.dtype], _p(out), x.shape[0],
                                         x.shape[1], ctypes.c_float(eps), _DT[out.dtype], self._s()), "add_rmsnorm")

    def add_rmsnorm_rows(self, x, delta, rows, weight, eps, out) -> None:
        self.launches += 1
        _check(self._core.sb_add_rmsnorm(_p(x), _p(delta), _p(rows), _p(weight), _DT[weight.dtype], _p(out), rows.shape[0],
                                         x.shape[1], ctypes.c_float(eps), _DT[out.dtype], self._s()), "add_rmsnorm_rows")

    def linear(self, a, w, out) -> None:
        """out[M,N] = a[M,K] @ w[N,K]^T (library matrix product)."""
        if a.dtype != w.dtype or a.shape[1] != w.shape[1] or out.shape[0] != a.shape[0] or out.shape[1] != w.shape[0]:
            raise KernelError(f"linear: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}, out {tuple(out.shape)} do not fit")
        m, n, k = a.shape[0], w.shape[0], a.shape[1]
        key = (a.dtype, out.dtype, m, n, k, self.use_skinny_linear, self.use_tcgen05, self.TCGEN05_MIN_TILES, self.tcgen05_for_plain_products, 0)
        route = self._routes.get(key)
        if route is None:
            route = 0
            if a.dtype == torch.bfloat16 and self.use_skinny_linear and self._core.sb_skinny_linear_supports(m, n, k, 0):
                route = 1
            elif (a.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and self.tcgen05_for_plain_products
                    and self._tcgen05_worthwhile(m, n) and self._core.sb_gemm_tcgen05_supports(m, n, k, 0)):
                route = 2
            elif (a.dtype == torch.float32 and out.dtype == torch.float32 and self.use_skinny_linear
                    and self._core.sb_skinny_linear_f32_supports(m, n, k)):
                route = 3
            self._routes[key] = route
        if route == 1:
            self.launches += 1
            _check(self._core.sb_skinny_linear(_p(a), _p(w), _p(out), m, n, k, _DT[out.dtype], 0, self._s()), "skinny linear")
        elif route == 2:
            self.launches += 1
            _check(self._core.sb_gemm_tcgen05(_p(a), _p(w), _p(out), m, n, k, 0, self._wait_flag(), self._s()), "tcgen05 product")
        elif route == 3:
            self.launches += 1
            _check(self._core.sb_skinny_linear_f32(_p(a), _p(w), _p(out), m, n, k, self._s()), "skinny linear, float32")
        else:
            self.library_calls += 1
            _check(self._gemm.sb_linear(_p(a), _p(w), _p(out), m, n, k, _DT[a.dtype], _DT[out.dtype], self._s()), "linear")

    def gate_up_swiglu(self, h, w_gate_up, out) -> None:
        """out[T, I] = silu(h @ w_gate^T) * (h @ w_up^T), w_gate_up = [w_gate; w_up] of shape [2I, K]."""
        t, inter, k = h.shape[0], out.shape[1], h.shape[1]
        if w_gate_up.shape[0] != 2 * inter or w_gate_up.shape[1] != k or out.shape[0] != t:
            raise KernelError("gate_up_swiglu: shapes do not fit")
        key = (h.dtype, out.dtype, t, inter, k, self.use_skinny_linear, self.use_tcgen05, self.TCGEN05_MIN_TILES, 1)
        route = self._routes.get(key)
        if route is None:
            route = 0
            if h.dtype == torch.bfloat16 and self.use_skinny_linear and self._core.sb_skinny_linear_supports(t, inter, k, 1):
                route = 1
            elif (h.dtype == torch.bfloat16 and self._tcgen05_worthwhile(t, 2 * inter)
                    and self._core.sb_gemm_tcgen05_supports(t, inter, k, 1)):
                route = 2
            self._routes[key] = route
        if route == 1:
            self.launches += 1
            _check(self._core.sb_skinny_linear(_p(h), _p(w_gate_up), _p(out), t, inter, k, _DT[out.dtype], 1, self._s()),
                   "skinny gate/up")
            return
        if route == 2:
            self.launches += 1
            _check(self._core.sb_gemm_tcgen05(_p(h), _p(w_gate_up), _p(out), t, inter, k, 1, self._wait_flag(), self._s()),
                   "tcgen05 gate/up")
            return
        gate_up = torch.empty((t, 2 * inter), dtype=h.dtype, device=h.device)
        self.linear(h, w_gate_up, gate_up)
        self.swiglu(gate_up, out)

    def swiglu(self, gate_up, out) -> None:
        self.launches += 1
        _check(self._core.sb_swiglu(_p(gate_up), _p(out), out.shape[0], out.shape[1], _DT[out.dtype], self._s()), "swiglu")

    def rope_cache_write(self, qkv, positions, token_row, inv_freq, pairing, rotary_dim, heads, kv_heads, head_dim,
                         k_cache, v_cache, block_table, page_size, write_cache) -> None:
        self.launches += 1
        num_pages = k_cache.shape[0] if k_cache is not None else 0
        _check(self._core.sb_rope_cache_write(
            _p(qkv), _p(positions), _p(token_row), _p(inv_freq), pairing, rotary_dim, heads, kv_heads, head_dim,
            _p(k_cache), _p(v_cache), _p(block_table), block_table.shape[1], page_size, num_pages,
            1 if write_cache else 0, _p(self.errors_tensor()), qkv.shape[0], _DT[qkv.dtype], self._s()), "rope_cache_write")

    def qkv_rope_cache(self, h, w_qkv, qkv, positions, token_row, inv_freq, pairing, rotary_dim, heads, kv_heads, head_dim,
                       k_cache, v_cache, block_table, page_size, write_cache, memo=None) -> None:
        """qkv = h @ w_qkv^T, queries and keys rotated, keys and values written to the cache pages.

        In bfloat16 with adjacent rotary pairs this is one kernel, for a handful of rows and for many (the product with
        rotation and cache write in its epilogue; only the query columns of ``qkv`` are then written). Otherwise, and
        for row counts in between that go to the library, the product and the rotary kernel run one after the other.
        ``memo``: a dict that lives as long as the step's positions do; what depends on them alone is kept there."""
        m, k = h.shape
        n = qkv.shape[1]
        if (h.dtype == torch.bfloat16 and self.use_skinny_linear and self.fuse_rope and pairing == 1 and head_dim % 8 == 0
                and self._core.sb_skinny_linear_supports(m, n, k, 0)):
            self.launches += 1
            _check(self._core.sb_skinny_qkv_rope(
                _p(h), _p(w_qkv), _p(qkv), m, k, _p(positions), _p(token_row), _p(inv_freq), rotary_dim, heads, kv_heads, head_dim,
                _p(k_cache), _p(v_cache), _p(block_table), block_table.shape[1], page_size, k_cache.shape[0],
                1 if write_cache else 0, _p(self.errors_tensor()), self._s()), "q/k/v product with rotation")
            return
        if (h.dtype == torch.bfloat16 and qkv.dtype == torch.bfloat16 and self.fuse_rope and pairing == 1
                and self._tcgen05_worthwhile(m, n)
                and self._core.sb_gemm_tcgen05_qkv_rope_supports(m, k, rotary_dim, heads, kv_heads, head_dim)):
            # many rows: the tensor-memory product with the same epilogue; cosines and sines from a table that the
            # first layer of the step makes and the others find in the step's memo
            key = ("rope_angles", inv_freq.data_ptr(), positions.data_ptr(), rotary_dim)
            angles = memo.get(key) if memo is not None else None
            if angles is None:
                angles = torch.empty((max(rotary_dim // 2, 1), m, 2), dtype=torch.float32, device=h.device)
                self.launches += 1
                _check(self._core.sb_rope_angles(_p(positions), _p(inv_freq), rotary_dim, m, _p(angles), self._s()), "rotary angles")
                if memo is not None:
                    memo[key] = angles
            self.launches += 1
            _check(self._core.sb_gemm_tcgen05_qkv_rope(
                _p(h), _p(w_qkv), _p(qkv), m, k, _p(positions), _p(token_row), _p(angles), rotary_dim, heads, kv_heads, head_dim,
                _p(k_cache), _p(v_cache), _p(block_table), block_table.shape[1], page_size, k_cache.shape[0],
                1 if write_cache else 0, _p(self.errors_tensor()), self._wait_flag(), self._s()),
                "tcgen05 q/k/v product with rotation")
            return
        self.linear(h, w_qkv, qkv)
        self.rope_cache_write(qkv, positions, token_row, inv_freq, pairing, rotary_dim, heads, kv_heads, head_dim,
                              k_cache, v_cache, block_table, page_size, write_cache)

    def attention(self, qkv, k_cache, v_cache, block_table, cu_q, kv_len, token_row, positions, heads, kv_heads, head_dim,
                  page_size, scale, window, out, shape) -> None:
        lib = self._attention_lib(head_dim)
        if qkv.dtype == torch.bfloat16 and not self.force_simt_attention:
            return self._attention_mma(lib, qkv, k_cache, v_cache, block_table, cu_q, kv_len, heads, kv_heads, head_dim,
                                       page_size, scale, window, out, shape)
        group = heads // kv_heads
        # requests of at most 16 rows run in the decoding shape, the others in tiles: one launch each, as needed
        self.launches += (1 if group <= 16 else 0) + (1 if group > 16 or shape.max_q * group > 16 else 0)
        _check(lib.sb_attention_simt(
            _p(qkv), qkv.shape[1], _p(k_cache), _p(v_cache), _p(block_table), block_table.shape[1], _p(cu_q), _p(kv_len),
            heads, kv_heads, page_size, k_cache.shape[0], ctypes.c_float(scale), window, _p(out), shape.rows, shape.max_q,
            _DT[qkv.dtype], self._s()), "attention")

    # Thread blocks of the deep shape that the key splits of a batch should fill: one per SM (set from the device's
    # SM count when the kernels are loaded; 148 on a B200).
    TARGET_BLOCKS = 148
    MAX_SPLITS = 32

    def split_plan(self, rows: int, kv_heads: int, max_kv: int) -> int:
        """Number of key splits of the deep shape for a batch; a function of sizes only, never of data.
        (Each request's own length is then shared out evenly over the splits inside the kernel.)"""
        want = max(1, self.TARGET_BLOCKS // max(1, rows * kv_heads))
        return max(1, min(want, -(-max_kv // 256), self.MAX_SPLITS))

    def _attention_mma(self, lib, qkv, k_cache, v_cache, block_table, cu_q, kv_len, heads, kv_heads, head_dim, page_size,
                       scale, window, out, shape) -> None:
        group = heads // kv_heads
        min_q = getattr(shape, "min_q", 1)
        which = 0
        if group > 16 or shape.max_q * group > 16:
            which |= 1
        if group <= 16 and min_q * group <= 16:
            which |= 2
            if group > 8 or (shape.max_q > 1 and min(shape.max_q, 16 // group) * group > 8):
                which |= 4      # some request of the deep shape may have more than 8 rows
                neg_q = getattr(shape, "neg_q_sorted", None)
                if neg_q is not None and group <= 8:
                    # the step says how many tokens each request brings: is any count in (8 // group, 16 // group]?
                    if bisect.bisect_left(neg_q, -(8 // group)) == bisect.bisect_left(neg_q, -(16 // group)):
                        which &= ~4
        # requests of the wide shape (more than 16 // group tokens): only they get blocks, if the step says who they are
        wide_rows, n_wide = None, 0
        neg_q = getattr(shape, "neg_q_sorted", None)
        if (which & 1) and neg_q is not None and getattr(shape, "rows_by_q", None) is not None:
            n_wide = bisect.bisect_left(neg_q, -(16 // group) if group <= 16 else 0)
            wide_rows = shape.rows_by_q
        num_splits, scratch, tickets = 1, None, None
        if which & 2:
            num_splits = self.split_plan(shape.rows, kv_heads, shape.max_kv)
            if num_splits > 1:
                scratch = self._scratch_buffer(lib, shape.rows, kv_heads, num_splits)
                tickets = self._ticket_buffer(shape.rows * kv_heads)
        if (which & 1) and self.use_tcgen05_attention and self._tc_attention_takes(lib, heads, kv_heads, head_dim, page_size, window, qkv.shape[1]):
            # prompt portions on the tensor-memory path; what is left (decoding rows) goes to the deep shape below
            self.launches += 1
            _check(lib.sb_attention_tc(
                _p(qkv), qkv.shape[1], qkv.shape[0], _p(k_cache), _p(v_cache), _p(block_table), block_table.shape[1], _p(cu_q),
                _p(kv_len), heads, kv_heads, page_size, k_cache.shape[0], ctypes.c_float(scale), _p(out),
                n_wide if wide_rows is not None else shape.rows, shape.max_q, _p(wide_rows), self._wait_flag(), self._s()),
                "tcgen05 attention")
            which &= ~1
            if not which:
                return
        self.launches += (which & 1) + ((which >> 1) & 1) + ((which >> 2) & 1)
        _check(lib.sb_attention_mma(
            _p(qkv), qkv.shape[1], _p(k_cache), _p(v_cache), _p(block_table), block_table.shape[1], _p(cu_q), _p(kv_len),
            heads, kv_heads, page_size, k_cache.shape[0], ctypes.c_float(scale), window, _p(out), shape.rows, shape.max_q,
            which, int(shape.max_kv), num_splits, _p(scratch), _p(tickets), _p(wide_rows), n_wide, self._s()), "attention")

    def _tc_attention_takes(self, lib, heads, kv_heads, head_dim, page_size, window, stride) -> bool:
        key = (heads, kv_heads, head_dim, page_size, window, stride)
        ok = self._tc_attention_ok.get(key)
        if ok is None:
            ok = self._tc_attention_ok[key] = bool(lib.sb_attention_tc_supports(heads, kv_heads, page_size, window, stride))
        return ok

    def _scratch_buffer(self, lib, rows: int, kv_heads: int, num_splits: int) -> torch.Tensor:
        """Float scratch for the partial results of split keys. Launches on one stream follow one another, so one buffer
        serves all layers and steps; a larger one is made when needed and the old one stays alive for captured graphs."""
        need = lib.sb_attention_mma_scratch_bytes(rows, kv_heads, num_splits) // 4
        if self._split_scratch is None or self._split_scratch.numel() < need:
            if self._split_scratch is not None:
                self._keep.append(self._split_scratch)
            self._split_scratch = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=self.device)
        return self._split_scratch

    def _ticket_buffer(self, n: int) -> torch.Tensor:
        """A zeroed int32 buffer of at least n entries. Every launch leaves it zeroed, so one buffer serves all
        layers and steps; a larger one is made when needed and the old ones stay alive for captured graphs."""
        if not self._tickets or self._tickets[-1].numel() < n:
            self._tickets.append(torch.zeros(max(n, 4096), dtype=torch.int32, device=self.device))
        return self._tickets[-1]

    # ---- whole layers of a decoding step in one launch ---------------------------------------------------------------
    def _stack_lib(self, head_dim: int):
        lib = self._stack.get(head_dim)
        if lib is None:
            job = layer_run_job(head_dim)
            job["verbose"] = self._verbose
            path = build.build_library(**job)
            self.paths[job["name"]] = path
            lib = self._stack[head_dim] = ctypes.CDLL(path)
            lib.sb_decode_stack_partial_floats.restype = ctypes.c_longlong
            if lib.sb_decode_stack_layer_bytes() != _STACK_LAYER.itemsize:
                raise KernelError("the layer table's layout on the host and in the library differ")
        return lib

    def plan_layer_run(self, descs):
        """(n, plan): the first n of the described layers can run as one launch in a decoding step (n may be 0).
        ``descs``: what Block.fused_description gives, one per layer in running order."""
        first = descs[0]
        if not self._layer_run_describable(first):
            return 0, None
        att, ff = first["mixer"], first["feed_forward"]
        key = (att["hidden"], att["heads"], att["kv_heads"], att["head_dim"], ff["intermediate"], att["page_size"])
        n = 0
        groups = []
        for d in descs:
            if not self._layer_run_describable(d):
                break
            a, f = d["mixer"], d["feed_forward"]
            if (a["hidden"], a["heads"], a["kv_heads"], a["head_dim"], f["intermediate"], a["page_size"]) != key:
                break
            if a["group"] not in groups:
                if len(groups) == _STACK_MAX_GROUPS:
                    break
                groups.append(a["group"])
            n += 1
        if n == 0:
            return 0, None
        hidden, heads, kv_heads, head_dim, inter, page_size = key
        lib = self._stack_lib(head_dim)
        blocks = lib.sb_decode_stack_blocks()
        if blocks <= 0 or not lib.sb_decode_stack_supports(1, hidden, heads, kv_heads, inter, blocks):
            return 0, None
        table = np.zeros(n, dtype=_STACK_LAYER)
        keep = []
        for i, d in enumerate(descs[:n]):
            a, f, n1, n2 = d["mixer"], d["feed_forward"], d["mixer_norm"], d["feed_forward_norm"]
            row = table[i]
            row["wqkv"], row["wo"] = a["w_qkv"].data_ptr(), a["w_o"].data_ptr()
            row["wgu"], row["wdown"] = f["w_gate_up"].data_ptr(), f["w_down"].data_ptr()
            row["norm1"], row["norm2"] = n1["weight"].data_ptr(), n2["weight"].data_ptr()
            row["inv_freq"] = a["inv_freq"].data_ptr()
            row["kc"], row["vc"] = a["k"].data_ptr(), a["v"].data_ptr()
            row["eps1"], row["eps2"] = n1["eps"], n2["eps"]
            row["scale_log2"] = a["scale"] * 1.4426950408889634
            row["rot"], row["window"] = a["rotary_dim"], a["window"]
            row["norm_f32"] = (1 if n1["weight"].dtype == torch.float32 else 0) | (2 if n2["weight"].dtype == torch.float32 else 0)
            row["group"] = groups.index(a["group"])
            row["num_pages"] = a["k"].shape[0]
            row["write_cache"] = 1 if a["writes"] else 0
            keep.extend([a["w_qkv"], a["w_o"], f["w_gate_up"], f["w_down"], n1["weight"], n2["weight"], a["inv_freq"], a["k"], a["v"]])
        dev_table = torch.from_numpy(table.view(np.uint8).copy()).to(self.device)
        return n, LayerRunPlan(lib, dev_table, keep, n, hidden, heads, kv_heads, head_dim, inter, groups, page_size, blocks)

    @staticmethod
    def _layer_run_describable(d) -> bool:
        if d is None or d.get("kind") != "pre_norm":
            return False
        a, f, n1, n2 = d.get("mixer"), d.get("feed_forward"), d.get("mixer_norm"), d.get("feed_forward_norm")
        if not (a and f and n1 and n2) or a.get("kind") != "attention" or f.get("kind") != "swiglu":
            return False
        if n1.get("kind") != "rms" or n2.get("kind") != "rms":
            return False
        if a["head_dim"] not in LAYER_RUN_HEAD_DIMS or a["w_qkv"].dtype != torch.bfloat16 or a["k"] is None or a["k"].dtype != torch.bfloat16:
            return False
        if a["rotary_dim"] > 0 and a["pairing"] != 1:
            return False
        if a["rotary_dim"] % 2 or n1["size"] != a["hidden"] or n2["size"] != a["hidden"] or f["hidden"] != a["hidden"]:
            return False
        return all(n["weight"].dtype in (torch.float32, torch.bfloat16) for n in (n1, n2))

    def layer_run_takes(self, plan: LayerRunPlan, ctx) -> bool:
        """Does this step go through the one-launch kernel? Decoding steps (one token per request) of at most 16 requests."""
        shape = ctx.shape
        if not (self.use_layer_runs and shape.pure_decode and shape.tokens <= _STACK_MAX_ROWS):
            return False
        ok = plan.takes.get(shape.tokens)
        if ok is None:
            ok = plan.takes[shape.tokens] = bool(plan.lib.sb_decode_stack_supports(shape.tokens, plan.hidden, plan.heads, plan.kv_heads,
                                                                                  plan.inter, plan.blocks))
        return ok

    def layer_run(self, plan: LayerRunPlan, x, pending, ctx):
        """Runs the plan's layers on the step's tokens: x [M, hidden] float32 is updated in place; returns (x, pending)."""
        m = x.shape[0]
        dev = x.device
        act = lambda cols: torch.empty((m, cols), dtype=torch.bfloat16, device=dev)
        n_qkv = (plan.heads + 2 * plan.kv_heads) * plan.head_dim
        x_scratch = torch.empty_like(x)
        delta_o, delta_down = act(plan.hidden), act(plan.hidden)
        qkv, attn, inter = act(n_qkv), act(plan.heads * plan.head_dim), act(plan.inter)
        num_splits = max(1, min(plan.blocks // max(1, m * plan.kv_heads), -(-ctx.shape.max_kv // 256), self.MAX_SPLITS))
        partials = tickets = None
        if num_splits > 1:
            need = plan.lib.sb_decode_stack_partial_floats(_STACK_MAX_ROWS, plan.kv_heads, self.MAX_SPLITS)
            if self._stack_partials is None or self._stack_partials.numel() < need:
                self._stack_partials = torch.empty(need, dtype=torch.float32, device=self.device)
                self._keep.append(self._stack_partials)
            partials = self._stack_partials
            tickets = self._ticket_buffer(m * plan.kv_heads)
        if self._stack_sync is None:
            self._stack_sync = torch.zeros(4, dtype=torch.int32, device=self.device)
        tables = (ctypes.c_void_p * _STACK_MAX_GROUPS)()
        widths = (ctypes.c_int * _STACK_MAX_GROUPS)()
        for i, g in enumerate(plan.groups):
            tables[i] = ctx.block_tables[g].data_ptr()
            widths[i] = ctx.block_tables[g].shape[1]
        self.launches += 1
        self.layer_runs += 1
        _check(plan.lib.sb_decode_stack(
            _p(plan.table), plan.n_layers, m, plan.hidden, plan.heads, plan.kv_heads, plan.inter, _p(ctx.positions), _p(ctx.kv_len),
            tables, widths, len(plan.groups), plan.page_size, _p(x), _p(x_scratch), _p(pending), _p(delta_o), _p(delta_down),
            _p(qkv), _p(attn), _p(inter), _p(partials), _p(tickets), num_splits, _p(self._stack_sync), _p(self.errors_tensor()),
            plan.blocks, _p(self.layer_run_timing), self._s()), "layers of a decoding step")
        return x, delta_down

    def sample(self, logits, temperature, req_ids, tok_index, seed, out, slots=None, last_token=None) -> None:
        self.launches += 1
        n = logits.shape[0]
        if self._sample_work is None or self._sample_work.numel() < 3 * n:
            # n 64-bit keys and n counters, zero now and after every call (kept alive for captured graphs)
            self._sample_work = torch.zeros(3 * max(n, 256), dtype=torch.int32, device=self.device)
            self._keep.append(self._sample_work)
        _check(self._core.sb_sample(_p(logits), _p(temperature), _p(req_ids), _p(tok_index), ctypes.c_ulonglong(seed),
                                    n, logits.shape[1], _p(out), _p(self._sample_work), _p(slots), _p(last_token), self._s()),
               "sample")


_INSTANCES: Dict[str, CudaKernels] = {}


def load_kernels(device="cuda:0", head_dims=(), verbose: bool = True) -> CudaKernels:
    """The kernels for ``device`` (one object per device; more head sizes are built when first used)."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available: this engine has no CPU path")
    key = str(torch.device(device))
    k = _INSTANCES.get(key)
    if k is None:
        k = _INSTANCES[key] = CudaKernels(device, head_dims, verbose)
    else:
        for d in head_dims:
            k._attention_lib(d)
    return k
