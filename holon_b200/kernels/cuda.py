"""The kernel table of the product path: hand-written CUDA for sm_100a, called through the library's C interface.

Every method takes torch tensors on one CUDA device, checks what the kernel assumes (device, dtype, contiguity,
shapes) and enqueues the kernel on torch's current stream. There is no other path: a size a kernel refuses raises
`KernelError` with the kernel's own message. Plain bfloat16 matrix products of more than 16 rows go to cuBLAS through
torch, as the reference's go through `torch.nn.functional.linear` (std/holon_std/ops/units.py:223-229); products
of up to 16 rows, SwiGLU's product with its activation, and float32 products run the library's own kernels.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .build import extension_path, library_path

_CODES = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16 tensors, not {t.dtype}") from None


class _ChainPhase(ctypes.Structure):
    """hb_chain_phase of csrc/api.h."""

    _fields_ = [(name, ctypes.c_void_p) for name in ("w", "x", "out", "h", "next_weight", "ss_out", "ss_in")] \
        + [(name, ctypes.c_int) for name in ("n", "k", "mode", "inter", "out_f32", "next_weight_f32", "parts_in", "dim_in")] \
        + [("next_offset", ctypes.c_float), ("eps_in", ctypes.c_float)]


class Extension:
    """The functions of a part's own CUDA library (`CudaKernels.extension`). `ext.call("fn", a, b, ...)` runs
    `int fn(a, b, ..., stream)` on torch's current stream after whatever the table still has queued, and raises
    `KernelError` with the library's text when it returns non-zero. `ptr`, `i32` and `check` are the table's own
    helpers for arguments: a tensor's address (0 for None), the same with the dtype checked, and device and contiguity."""

    def __init__(self, kernels: "CudaKernels", name: str, path, status_mirrors=()) -> None:
        self.kernels, self.name, self.path = kernels, name, path
        self.lib = ctypes.CDLL(str(path))
        self._fn: dict = {}
        self.ptr, self.i32, self.check = kernels._p, kernels._i32, kernels._check
        for fn in status_mirrors:             # its bounded waits report into the word that the engine reads
            word = ctypes.POINTER(ctypes.c_uint)()
            with torch.cuda.device(kernels.device):
                if kernels.lib.hb_status_word_device(ctypes.byref(word)) or getattr(self.lib, fn)(word):
                    raise KernelError(f"{name}.{fn}: {kernels.lib.hb_last_error().decode()}")

    def call(self, fn: str, *args) -> None:
        self.kernels._call_in(self.lib, self._fn, fn, *args)


class CudaKernels:
    name = "cuda sm_100a"

    def __init__(self, device) -> None:
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError(f"the engine runs on a CUDA device; {self.device} is none")
        self.path = library_path()
        self.lib = ctypes.CDLL(str(self.path), mode=ctypes.RTLD_GLOBAL)      # (extensions use its hb_set_error)
        self._extensions: dict[str, Extension] = {}
        self.lib.hb_last_error.restype = ctypes.c_char_p
        self._fn = {}
        self._index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        self.launches = 0
        self._splits: dict = {}
        # Which kernel attends for rows of several tokens: "tcgen05" (csrc/attention_tcgen05.cu, for head size 128 and
        # pages of a multiple of 64 tokens; every other shape takes the mma.sync kernel) or "mma" (mma.sync always:
        # any head size up to 256 in steps of 16, any page size).
        self.prefill_attention = os.environ.get("HOLON_B200_PREFILL_ATTENTION", "tcgen05")
        if self.prefill_attention not in ("mma", "tcgen05"):
            raise KernelError(f"HOLON_B200_PREFILL_ATTENTION must be mma or tcgen05, not {self.prefill_attention!r}")
        # Which kernel multiplies bfloat16 matrices of more than SKINNY_ROWS rows: "auto" (the default: the library
        # through torch, as the reference uses one there, except SwiGLU's gate/up product, which goes to the
        # hand-written tcgen05 kernel with the activation in its epilogue where that is faster than the library's
        # product plus an activation kernel), "cublas" (the library always) or "tcgen05" (csrc/gemm_tcgen05*.cu always).
        self.gemm = os.environ.get("HOLON_B200_GEMM", "auto")
        if self.gemm not in ("auto", "cublas", "tcgen05"):
            raise KernelError(f"HOLON_B200_GEMM must be auto, cublas or tcgen05, not {self.gemm!r}")
        self.gemm_pair = os.environ.get("HOLON_B200_GEMM_PAIR", "1") != "0"   # the tcgen05 product by CTA pairs
        self.attention_bf16 = "fast"          # "generic" forces the CUDA-core kernel for bfloat16 too (tests)
        # How the keys of rows that bring one token are shared out when one CTA per (row, kv head) is too few:
        # "splits" (every row cut into the same number of parts), "balanced" (every CTA of one GPU-filling wave takes
        # the same number of 64-key tiles, whatever the rows' lengths) or "auto" (balanced for a batch with one row far
        # longer than the others, where equal cuts leave most CTAs with almost nothing; see decode_mode).
        self.decode_attention = os.environ.get("HOLON_B200_DECODE_ATTENTION", "auto")
        if self.decode_attention not in ("auto", "balanced", "splits"):
            raise KernelError(f"HOLON_B200_DECODE_ATTENTION must be auto, balanced or splits, not {self.decode_attention!r}")
        self.decode_cluster = os.environ.get("HOLON_B200_DECODE_CLUSTER", "1") != "0"   # splits of up to 16 merge in the kernel
        self.fused_qkv = os.environ.get("HOLON_B200_FUSED_QKV", "1") != "0"   # decode steps: norm, rotation, cache write in the product
        self.fused_norm = os.environ.get("HOLON_B200_FUSED_NORM", "1") != "0"   # decode steps: residual sum and next norm in the product before
        # Where csrc/gemm_mid.cu (tcgen05, the k range split over a thread-block cluster) runs (HOLON_B200_MID). "auto", the
        # default, for weights of 32 MB or more: SwiGLU's product at up to MID_ROWS rows (one CTA a tile, no sum over a
        # cluster; its idle warps add up the row scales while the weights stream, which costs the mma.sync kernel a trip
        # to the L2 at the end of every CTA: back to back in a graph on rows that lack their norm's scale, Qwen3-8B
        # sizes, 36.3 us against 38.0 at 8 rows, 36.3 against 37.4 at 1, 36.5 against 42.3 at 16; from 17 rows level
        # with the library's product, and the activation kernel is saved), and the attention's first product at 9 to
        # 16 rows (14.4 us against 15.1 at 16 rows: the mma.sync kernel reads x for a second tile of eight rows there;
        # at 8 rows it is 13.9 against 14.1 the other way). o_proj and down stay with the mma.sync kernel up to 16 rows
        # (8.5 and 18.6 us against 10.3 and 20.6: a launch of this kernel costs 5 us before its first byte counts, the
        # other 2). "all": steps of 17 to MID_ROWS rows keep every fused product there, instead of the library's
        # product and kernels of their own for the work around it; "swiglu": of those only SwiGLU's, whatever the
        # weight's size. Measured, decode steps of 64 / 32 / 17 rows at 2,304 keys: 7.31 / 5.25 / 4.46 ms with the library
        # alone, 7.24 / 5.24 / 4.45 with SwiGLU's product here, 7.48 / 5.28 / 4.48 with "all" (a clustered product costs
        # 3 us more than the library's, which is what the kernels it saves cost). "0": never. `mid_split`: tests force
        # the cluster size (0: chosen per launch).
        self.mid_mode = os.environ.get("HOLON_B200_MID", "auto")
        if self.mid_mode not in ("0", "auto", "swiglu", "all"):
            raise KernelError(f"HOLON_B200_MID must be 0, auto, swiglu or all, not {self.mid_mode!r}")
        self.mid_split = 0
        self.mid_launches = 0
        self.mid_min_rows = int(os.environ.get("HOLON_B200_MID_MIN_ROWS", "9"))   # the attention's first product: fewer rows stay with the mma.sync kernel
        # Steps of 17 to WIDE_ROWS rows and weights below MID_WEIGHT elements (small models, where a kernel is its launch):
        # the mma.sync kernel with four tiles of x a warp keeps the fused epilogues ("1"), or the library multiplies and
        # kernels of their own do the rest ("0").
        self.skinny32 = os.environ.get("HOLON_B200_SKINNY32", "1") != "0"
        self.sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.decode_ctas = None               # tests: a fixed number of CTAs for the balanced kernel
        self.latent_split = None              # tests: a fixed number of key parts for one-token rows of latent attention
        # The experts' products in bfloat16: "fast" (the default: tcgen05 for prompts, mma.sync tiles or the CUDA-core
        # kernel for fewer rows an expert), "mma" (never tcgen05), "tcgen05" (always), "generic" (the kernel of any dtype).
        self.expert_products = os.environ.get("HOLON_B200_EXPERTS", "fast")
        if self.expert_products not in ("fast", "mma", "tcgen05", "generic"):
            raise KernelError(f"HOLON_B200_EXPERTS must be fast, mma, tcgen05 or generic, not {self.expert_products!r}")
        self.expert_tile_rows = 0             # tests: 16, 64 or 128 rows a tile of the experts' tensor-core products (0: chosen)
        self.prefill_tile = None              # tests, microbench: 128 or 256 queries a CTA of the tcgen05 prefill kernel
        # Decode steps: the products of a layer that follow one another on the same few rows (the mixer's last, the
        # feed-forward's two, the next mixer's first) can be queued and run in one launch; every other call of this table
        # runs what is queued first. HOLON_B200_CHAIN: "tickets" (csrc/gemm_tickets.cu: every CTA a tile of one of the
        # products, drawn in order, so that a product starts while the one before ends), "ring" (csrc/gemm_chain.cu: one
        # persistent kernel with a shared-memory ring; slower as measured) or "0" (every product its own launch).
        self.chain = {"0": "", "1": "tickets"}.get(os.environ.get("HOLON_B200_CHAIN", "0"), os.environ.get("HOLON_B200_CHAIN", "0"))
        if self.chain not in ("", "tickets", "ring"):
            raise KernelError(f"HOLON_B200_CHAIN must be 0, tickets or ring, not {self.chain!r}")
        self.chain_cooperative = os.environ.get("HOLON_B200_CHAIN_COOPERATIVE", "1") != "0"
        self._pending: list = []              # (phase, tensors it names) of products queued, in order
        self.chain_launches = self.chain_phases = 0
        self.lib.hb_gemm_chain_capacity.restype = ctypes.c_int
        with torch.cuda.device(self.device):
            self._chain_slots = int(self.lib.hb_gemm_chain_capacity())
        if self._chain_slots < 1:
            raise KernelError("hb_gemm_chain_capacity: the device runs no CTA of the chained products' kernel")
        self._chain_sync = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._chain_flags = torch.zeros(self._chain_slots, dtype=torch.int32, device=self.device)
        self._chain_scratch = torch.empty(self._chain_slots * 512, dtype=torch.float32, device=self.device)
        self._ticket_state = torch.zeros(8, dtype=torch.int32, device=self.device)
        # One word of page-locked host memory that a kernel's bounded wait writes when it gives up (csrc/status.cu)
        word = ctypes.POINTER(ctypes.c_uint)()
        with torch.cuda.device(self.device):
            if self.lib.hb_status_word(ctypes.byref(word)):
                raise KernelError(f"hb_status_word: {self.lib.hb_last_error().decode()}")
        self._status_word = word

    # ------------------------------------------------------------------ plumbing
    @property
    def mid(self) -> bool:
        """Whether steps of 17 to MID_ROWS rows keep their fused products (csrc/gemm_mid.cu)."""
        return self.mid_mode == "all"

    WIDE_ROWS = 32                            # rows the mma.sync kernel takes with four tiles of x a warp

    def _wide_takes(self, m: int, weight, stride: int | None = None) -> bool:
        """Whether a product of 17 to WIDE_ROWS rows with a small `weight` runs in the 32-row mma.sync kernel (`stride`:
        the tokens a part of its rows' partial sums holds, if the rows are parts.base.Scaled: that kernel reads 32)."""
        return self.skinny32 and self.SKINNY_ROWS < m <= self.WIDE_ROWS and weight.numel() < self.MID_WEIGHT \
            and stride in (None, self.WIDE_ROWS) and not (self.mid_mode == "all" and stride is None)

    MID_WEIGHT = 16 << 20                     # elements of a weight from which "auto" sends a product to csrc/gemm_mid.cu

    def _mid_takes(self, m: int, weight, mode: int) -> bool:
        """Whether the product of `m` rows with `weight` and the epilogue `mode` (1 SwiGLU, 2 q/k norm, rotation and
        cache write) runs in csrc/gemm_mid.cu rather than in the kernel for up to SKINNY_ROWS rows."""
        if self.mid_mode == "0" or m > self.MID_ROWS or (self.chain and m <= self.SKINNY_ROWS):
            return False                                   # (chained products are the mma.sync kernel's tiles)
        large = weight.numel() >= self.MID_WEIGHT
        if m <= self.SKINNY_ROWS:                          # SwiGLU's at any number of rows, the attention's first from 9 on
            return large and (mode == 1 or (mode == 2 and m >= self.mid_min_rows))
        return self.mid_mode == "all" or (mode == 1 and (self.mid_mode == "swiglu" or (large and self.gemm != "cublas")))

    def _call(self, name: str, *args) -> None:
        if self._pending:                      # what is queued comes first: this call may read what it writes
            self.flush()
        self._launch(name, *args)

    def _launch(self, name: str, *args) -> None:
        fn = self._fn.get(name)
        if fn is None:
            fn = self._fn[name] = getattr(self.lib, name)
            fn.restype = ctypes.c_int
        code = fn(*args, ctypes.c_void_p(self._stream()))
        self.launches += 1
        if code:
            raise KernelError(f"{name}: {self.lib.hb_last_error().decode()}")

    def _call_in(self, lib, cache: dict, name: str, *args) -> None:
        """`_call` for a function of another library (an extension's)."""
        if self._pending:
            self.flush()
        fn = cache.get(name)
        if fn is None:
            try:
                fn = cache[name] = getattr(lib, name)
            except AttributeError:
                raise KernelError(f"{name}: the extension's library exports no such function") from None
            fn.restype = ctypes.c_int
        code = fn(*args, ctypes.c_void_p(self._stream()))
        self.launches += 1
        if code:
            raise KernelError(f"{name}: {self.lib.hb_last_error().decode() or f'returned {code}'}")

    def extension(self, name: str, sources, build_dir=None, status_mirrors=()) -> Extension:
        """A part's own CUDA files as a library beside this one: compiled on first use (kernels/build.py:
        `extension_path`), loaded once per table. The part calls its functions through the `Extension` it gets; this
        file, api.h and the main library stay as they are. `status_mirrors`: the names its files gave to
        HB_DEFINE_STATUS_MIRROR (csrc/tcgen05.cuh), one per file with bounded waits; `status()` then shows a wait of
        theirs that gave up, and the engine stops on it as on any other."""
        ext = self._extensions.get(name)
        if ext is None:
            path = extension_path(name, sources, build_dir)
            ext = self._extensions[name] = Extension(self, name, path, status_mirrors)
        return ext

    # ---- products queued for one persistent kernel (decode steps)
    MAX_CHAIN = 8                              # phases a launch takes (csrc/gemm_chain.cu)
    MAX_TICKETS = 4                            # products a launch takes (csrc/gemm_tickets.cu)

    def _queue(self, *, w, x, out, mode: int, n: int, inter: int = 0, h=None, next_weight=None, next_offset: float = 0.0,
               ss_out=None, scaled=None) -> None:
        if len(self._pending) >= (self.MAX_CHAIN if self.chain == "ring" else self.MAX_TICKETS):
            self.flush()
        y = scaled.y if scaled is not None else x
        phase = _ChainPhase(w=w.data_ptr(), x=y.data_ptr(), out=out.data_ptr(), h=h.data_ptr() if h is not None else None,
                            next_weight=next_weight.data_ptr() if next_weight is not None else None,
                            ss_out=ss_out.data_ptr() if ss_out is not None else None,
                            ss_in=scaled.ss.data_ptr() if scaled is not None else None, n=n, k=y.shape[1], mode=mode,
                            inter=inter, out_f32=int(out.dtype == torch.float32),
                            next_weight_f32=int(next_weight is not None and next_weight.dtype == torch.float32),
                            parts_in=scaled.ss.shape[0] if scaled is not None else 0,
                            dim_in=scaled.dim if scaled is not None else 0, next_offset=float(next_offset),
                            eps_in=float(scaled.eps) if scaled is not None else 0.0)
        keep = (w, x, out, h, next_weight, ss_out, scaled)            # (the tensors stay alive until the launch)
        if self._pending and self._pending[0][2] != y.shape[0]:
            self.flush()
        self._pending.append((phase, keep, y.shape[0]))

    def flush(self) -> None:
        """Launches what is queued: one persistent kernel for all of it. Everything this table's other calls do comes
        after it; whoever reads a queued product's output by other means (torch operations) calls this first."""
        if not self._pending:
            return
        pending, self._pending = self._pending, []
        phases = (_ChainPhase * len(pending))(*[p for p, _, _ in pending])
        if self.chain == "ring":
            self._launch("hb_gemm_chain", phases, len(pending), pending[0][2], self._p(self._chain_sync),
                         self._p(self._chain_scratch), self._p(self._chain_flags), self._chain_slots, int(self.chain_cooperative))
        else:
            self._launch("hb_gemm_tickets", phases, len(pending), pending[0][2], self._p(self._ticket_state))
        self.chain_launches += 1
        self.chain_phases += len(pending)

    def _chains(self, m: int, k: int, *tensors) -> bool:
        """Whether a product of `m` rows over `k` columns of these bfloat16 tensors may be queued."""
        return bool(self.chain) and 0 < m <= self.SKINNY_ROWS and k % 8 == 0 \
            and all(t.dtype == torch.bfloat16 and t.data_ptr() % 16 == 0 for t in tensors)

    def _stream(self) -> int:
        """The handle of torch's current stream on the device (a few hundred kernels a step ask for it)."""
        if self._raw_stream is not None:
            return self._raw_stream(self._index)
        return torch.cuda.current_stream(self.device).cuda_stream

    def _check(self, *tensors: torch.Tensor | None) -> None:
        index = self._index
        for t in tensors:
            if t is None or (t.is_cuda and t.get_device() == index and t.is_contiguous()):
                continue
            if t.device != self.device:
                raise KernelError(f"a tensor lives on {t.device}, the kernels run on {self.device}")
            raise KernelError(f"kernels take contiguous tensors; got strides {t.stride()} for shape {tuple(t.shape)}")

    @staticmethod
    def _p(t: torch.Tensor | None) -> ctypes.c_void_p:
        return ctypes.c_void_p(t.data_ptr() if t is not None else 0)

    @staticmethod
    def _i32(t: torch.Tensor | None, what: str) -> ctypes.c_void_p:
        if t is not None and t.dtype != torch.int32:
            raise KernelError(f"{what} must be int32, not {t.dtype}")
        return ctypes.c_void_p(t.data_ptr() if t is not None else 0)

    # ------------------------------------------------------------------ kernels
    def embed(self, out, table, ids) -> None:
        self._check(out, table, ids)
        if out.dtype != torch.float32 or out.shape != (ids.shape[0], table.shape[1]):
            raise KernelError("embed: out must be float32 [tokens, hidden]")
        self._call("hb_embed", self._p(out), self._p(table), _code(table), self._i32(ids, "ids"),
                   ids.shape[0], table.shape[1], table.shape[0])

    def rmsnorm(self, out, x, weight, eps, offset) -> None:
        self._check(out, x, weight)
        if out.shape != x.shape or weight.shape != (x.shape[-1],):
            raise KernelError("rmsnorm: out and x must have one shape, weight [dim]")
        rows = x.numel() // x.shape[-1]
        self._call("hb_add_rmsnorm", self._p(out), _code(out), self._p(x), _code(x), self._p(None), self._p(weight),
                   _code(weight), ctypes.c_float(eps), ctypes.c_float(offset), self._p(None), rows, x.shape[-1])

    def add_rmsnorm(self, out, h, delta, weight, eps, offset, index) -> None:
        self._check(out, h, delta, weight, index)
        rows = index.shape[0] if index is not None else h.shape[0]
        if h.dtype != torch.float32 or out.shape != (rows, h.shape[1]) or weight.shape != (h.shape[1],):
            raise KernelError("add_rmsnorm: h must be float32 [tokens, dim], out [rows, dim], weight [dim]")
        if delta is not None and (delta.shape != h.shape or delta.dtype != out.dtype):
            raise KernelError("add_rmsnorm: delta must have h's shape and out's dtype")
        self._call("hb_add_rmsnorm", self._p(out), _code(out), self._p(h), 0, self._p(delta), self._p(weight),
                   _code(weight), ctypes.c_float(eps), ctypes.c_float(offset), self._i32(index, "index"), rows,
                   h.shape[1])

    def silu_mul(self, out, gate_up) -> None:
        self._check(out, gate_up)
        if gate_up.shape != (out.shape[0], 2 * out.shape[1]) or out.dtype != gate_up.dtype:
            raise KernelError("silu_mul: gate_up must be [tokens, 2 * inter] of out's dtype")
        self._call("hb_silu_mul", self._p(out), self._p(gate_up), _code(out), out.shape[0], out.shape[1])

    def qk_norm_rope_kv_write(self, q_out, qkv, positions, table, rotary_dim, q_weight, k_weight, eps, offset, kv,
                              write_index, heads, kv_heads, head_dim, bias=None) -> None:
        """`bias` (qkv's dtype, [(heads + 2 kv_heads) head_dim], or None) is added to q, k and v first."""
        self._check(q_out, qkv, positions, table, q_weight, k_weight, kv, write_index, bias)
        t = qkv.shape[0]
        if bias is not None and (bias.shape != (qkv.shape[1],) or bias.dtype != qkv.dtype):
            raise KernelError("qk_norm_rope_kv_write: bias must be one row of qkv's width and dtype")
        if qkv.shape != (t, (heads + 2 * kv_heads) * head_dim) or q_out.shape != (t, heads, head_dim) \
                or q_out.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_kv_write: qkv must be [tokens, (heads + 2 kv_heads) head_dim], q_out "
                              "[tokens, heads, head_dim], of one dtype")
        if table is not None and (table.dtype != torch.float32 or table.shape[1] != rotary_dim):
            raise KernelError("qk_norm_rope_kv_write: the rotation table must be float32 [positions, rotary_dim]")
        if kv is not None and (kv.dtype != qkv.dtype or kv.shape[1:3] != (2, kv_heads) or kv.shape[4] != head_dim):
            raise KernelError("qk_norm_rope_kv_write: kv must be [pages, 2, kv_heads, page_size, head_dim] of qkv's dtype")
        self._call("hb_qk_norm_rope_kv_write", self._p(q_out), self._p(qkv), _code(qkv),
                   self._i32(positions, "positions"), self._p(table), rotary_dim,
                   table.shape[0] if table is not None else 0, self._p(q_weight), self._p(k_weight),
                   _code(q_weight) if q_weight is not None else 0, ctypes.c_float(eps), ctypes.c_float(offset),
                   self._p(kv), self._i32(write_index, "write_index"), kv.shape[0] if kv is not None else 0,
                   kv.shape[3] if kv is not None else 1, t, heads, kv_heads, head_dim, self._p(bias))

    def qkv_rope(self, q_out, x, weight, positions, table, rotary_dim, q_weight, k_weight, eps, offset, kv,
                 write_index, heads, kv_heads, head_dim) -> bool:
        """The product x · weightᵀ with qk_norm_rope_kv_write folded into its epilogue, for the few rows of a decode
        step (one kernel instead of two). False, with nothing done, where that kernel does not apply: more than
        SKINNY_ROWS rows, another dtype, a head size other than 32, 64 or 128, a partial rotation or none."""
        scaled, x = (x, x.y) if hasattr(x, "ss") else (None, x)      # rows that lack their norm's scale (parts.base.Scaled)
        t, k = x.shape
        wide = x.dtype == torch.bfloat16 and self._wide_takes(t, weight, scaled.ss.shape[1] if scaled else None)
        if not self.fused_qkv or x.dtype != torch.bfloat16 or (t > (self.MID_ROWS if self.mid else self.SKINNY_ROWS) and not wide) or k % 8 or table is None \
                or head_dim not in (32, 64, 128) or rotary_dim != head_dim or (q_weight is None) != (k_weight is None):
            return False
        self._check(q_out, x, weight, positions, table, q_weight, k_weight, kv, write_index)
        if weight.shape != ((heads + 2 * kv_heads) * head_dim, k) or weight.dtype != x.dtype \
                or q_out.shape != (t, heads, head_dim) or q_out.dtype != x.dtype:
            raise KernelError("qkv_rope: w must be [(heads + 2 kv_heads) head_dim, k] and q_out [tokens, heads, head_dim], bfloat16")
        if table.dtype != torch.float32 or table.shape[1] != head_dim:
            raise KernelError("qkv_rope: the rotation table must be float32 [positions, head_dim]")
        if kv is not None and (kv.dtype != x.dtype or kv.shape[1:3] != (2, kv_heads) or kv.shape[4] != head_dim):
            raise KernelError("qkv_rope: kv must be [pages, 2, kv_heads, page_size, head_dim], bfloat16")
        if q_weight is not None and q_weight.dtype != k_weight.dtype:
            raise KernelError("qkv_rope: the two norm weights must have one dtype")
        if wide:
            self._call("hb_qkv_rope_skinny32", self._p(q_out), self._p(x), self._p(weight), t, k,
                       self._i32(positions, "positions"), self._p(table), table.shape[0], self._p(q_weight), self._p(k_weight),
                       int(q_weight is not None and q_weight.dtype == torch.float32), ctypes.c_float(eps),
                       ctypes.c_float(offset), self._p(kv), self._i32(write_index, "write_index"),
                       kv.shape[0] if kv is not None else 0, kv.shape[3] if kv is not None else 1, heads, kv_heads, head_dim,
                       self._p(scaled.ss) if scaled else None, scaled.ss.shape[0] if scaled else 0,
                       ctypes.c_float(scaled.eps if scaled else 0.0), scaled.dim if scaled else 0)
            return True
        if t > self.SKINNY_ROWS or self._mid_takes(t, weight, 2):
            self.mid_launches += 1
            self._call("hb_qkv_rope_mid", self._p(q_out), self._p(x), self._p(weight), t, k,
                       self._i32(positions, "positions"), self._p(table), table.shape[0], self._p(q_weight), self._p(k_weight),
                       int(q_weight is not None and q_weight.dtype == torch.float32), ctypes.c_float(eps),
                       ctypes.c_float(offset), self._p(kv), self._i32(write_index, "write_index"),
                       kv.shape[0] if kv is not None else 0, kv.shape[3] if kv is not None else 1, heads, kv_heads, head_dim,
                       self._p(scaled.ss) if scaled else None, scaled.ss.shape[0] if scaled else 0,
                       scaled.ss.shape[1] if scaled else 0, ctypes.c_float(scaled.eps if scaled else 0.0),
                       scaled.dim if scaled else 0, int(self.mid_split))
            return True
        if self._pending and scaled is not None and self._chains(t, k, x, weight):
            # the product that made these rows is still queued: this one joins it as a plain product, so that the
            # weights of both stream through one kernel, and the norm, rotation and cache write run behind it
            qkv = torch.empty((t, weight.shape[0]), dtype=torch.bfloat16, device=self.device)
            self._queue(w=weight, x=x, out=qkv, mode=0, n=weight.shape[0], scaled=scaled)
            self.qk_norm_rope_kv_write(q_out, qkv, positions, table, rotary_dim, q_weight, k_weight, eps, offset, kv,
                                       write_index, heads, kv_heads, head_dim)
            return True
        self._call("hb_qkv_rope_skinny_linked", self._p(q_out), self._p(x), self._p(weight), t, k,
                   self._i32(positions, "positions"), self._p(table), table.shape[0], self._p(q_weight), self._p(k_weight),
                   int(q_weight is not None and q_weight.dtype == torch.float32), ctypes.c_float(eps),
                   ctypes.c_float(offset), self._p(kv), self._i32(write_index, "write_index"),
                   kv.shape[0] if kv is not None else 0, kv.shape[3] if kv is not None else 1, heads, kv_heads, head_dim,
                   self._p(scaled.ss) if scaled else None, scaled.ss.shape[0] if scaled else 0,
                   ctypes.c_float(scaled.eps if scaled else 0.0), scaled.dim if scaled else 0)
        return True

    def paged_attention(self, out, q, kv, block_table, rows, scale, window, sinks=None) -> None:
        """`sinks` (float32 [heads], or None): a weight exp(sinks[h]) in each head's softmax denominator that has
        neither key nor value. Every kernel takes them but the balanced form for one-token rows (such rows then run
        with equal cuts, merged in a cluster or by the merge kernel)."""
        self._check(out, q, kv, block_table, rows.row_slot, rows.query_start, rows.kv_len, sinks)
        t, heads, head_dim = q.shape
        if sinks is not None and (sinks.dtype != torch.float32 or sinks.shape != (heads,)):
            raise KernelError("paged_attention: sinks must be float32 [heads]")
        if out.shape != q.shape or kv.dtype != q.dtype or out.dtype != q.dtype or kv.shape[4] != head_dim:
            raise KernelError("paged_attention: out and q [tokens, heads, head_dim], kv [pages, 2, kv_heads, page_size, "
                              "head_dim], one dtype")
        fast = q.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256 and self.attention_bf16 == "fast"
        if not fast:
            return self._attention_generic(out, q, kv, block_table, rows, scale, window, sinks)
        kv_heads = kv.shape[2]
        common = (self._i32(block_table, "block_table"), block_table.shape[1], self._i32(rows.row_slot, "row_slot"),
                  self._i32(rows.query_start, "query_start"), self._i32(rows.kv_len, "kv_len"))
        sizes = (heads, kv_heads, head_dim, kv.shape[0], kv.shape[3], ctypes.c_float(scale), int(window))
        if rows.n_decode:
            splits = self.decode_splits(rows.n_decode, heads, kv_heads, rows.max_kv)
            mode = self._decode_mode_of(rows)
            if sinks is None and splits > 1 and mode == "balanced" and rows.n_decode <= self.BALANCED_ROWS:
                pairs = rows.n_decode * kv_heads * (-(-(heads // kv_heads) // 16))
                slots = self.sms * (1 if head_dim > 128 else 3)       # CTAs of this kernel that one wave holds
                if 2 * pairs <= slots:                                # a whole number of CTAs per (row, kv head): rows of
                    slots = pairs * (slots // pairs)                  # equal length are then cut at their own ends only
                # (with more than half a wave of pairs that rounding would leave one CTA a pair and up to half of the
                # GPU idle: 29 rows of 8 kv heads, 83 µs against 50 µs with equal cuts)
                ctas = self.decode_ctas or max(1, min(slots, pairs * (-(-rows.max_kv // 64)) // 2))
                floats = (ctas + pairs) * min(16, heads // kv_heads) * (head_dim + 2)
                scratch = torch.empty(floats, dtype=torch.float32, device=self.device)
                self._call("hb_attention_decode_bf16_balanced", self._p(out), self._p(scratch), self._p(q), self._p(kv),
                           *common, rows.n_decode, *sizes, ctas)
            elif splits > 1 and (few := self.decode_cluster_splits(rows.n_decode, heads, kv_heads, head_dim,
                                                                   rows.max_kv, splits)):
                self._call("hb_attention_decode_bf16_cluster", self._p(out), self._p(q), self._p(kv), *common,
                           rows.n_decode, *sizes, few, self._p(sinks))
            else:
                floats = rows.n_decode * heads * splits * (head_dim + 2) if splits > 1 else 0
                scratch = torch.empty(floats, dtype=torch.float32, device=self.device) if floats else None
                self._call("hb_attention_decode_bf16", self._p(out), self._p(scratch), self._p(q), self._p(kv), *common,
                           rows.n_decode, *sizes, splits, self._p(sinks))
        if rows.n_rows > rows.n_decode:
            if self.prefill_attention == "tcgen05" and head_dim == 128 and kv.shape[3] % 64 == 0:
                tile_q, tiles = 256, self._query_tiles(rows, 256)
                if self.prefill_tile == 128 or (self.prefill_tile is None and 4 * heads * tiles < 3 * self.sms):              # tiles of 256 queries would leave SMs idle: one group of
                    tile_q, tiles = 128, self._query_tiles(rows, 128)   # 128 a CTA, twice the CTAs
                self._call("hb_attention_prefill_tcgen05", self._p(out), self._p(q), self._p(kv), *common,
                           rows.n_decode, rows.n_rows, tiles, t, *sizes, tile_q, self._p(sinks))
            else:
                self._call("hb_attention_prefill_bf16", self._p(out), self._p(q), self._p(kv), *common, rows.n_decode,
                           rows.n_rows, self._query_tiles(rows, 64), *sizes, self._p(sinks))

    KV_BUCKET_MIN = 512                       # the smallest number of keys a captured decode launch is planned for

    def attention_capture_plan(self, rows, max_model_len: int):
        """For a step that runs as a CUDA graph: what of the attention's launch plan a captured launch keeps, as a
        hashable key, pinned on `rows` so that every layer's launch is planned with it. The keys of a row are cut for
        a power-of-two bucket of the longest row (a graph of that bucket serves every batch whose longest row fits
        it; planning every graph for the longest request the engine takes would cut 2,000-token rows like 8,000-token
        ones), the one-token rows' keys are shared out in the mode their lengths call for, and rows of several tokens
        get the most query tiles any cut of their tokens into that many rows can have (tiles beyond a step's own exit
        at once)."""
        lens = rows.host_kv_len
        bucket = self.KV_BUCKET_MIN
        longest = int(lens.max()) if lens is not None and len(lens) else max_model_len
        while bucket < longest:
            bucket *= 2
        bucket = min(bucket, max(max_model_len, longest))
        mode = self.decode_mode(lens[:rows.n_decode] if lens is not None else None) if rows.n_decode else None
        rows.max_kv = bucket
        rows.plan["mode"] = mode
        portions, tokens = rows.n_rows - rows.n_decode, rows.n_tokens - rows.n_decode
        for size in (64, 128, 256):
            rows.plan[size] = tokens // size + portions
        return mode, bucket

    # Every layer of a step asks the same questions about the step's rows: the answers are kept on the rows.
    def _decode_mode_of(self, rows) -> str:
        plan = rows.plan
        if "mode" not in plan:
            lens = rows.host_kv_len[:rows.n_decode] if rows.host_kv_len is not None else None
            plan["mode"] = self.decode_mode(lens)
        return plan["mode"]

    @staticmethod
    def _query_tiles(rows, size: int) -> int:
        """Tiles of `size` queries over the rows that bring several tokens."""
        plan = rows.plan
        if size not in plan:
            qs = rows.host_query_start
            plan[size] = sum((int(qs[b + 1]) - int(qs[b]) + size - 1) // size for b in range(rows.n_decode, rows.n_rows))
        return plan[size]

    BALANCED_ROWS = 256                       # rows the balanced decode kernel takes (its prefix array)

    def decode_mode(self, kv_lens) -> str:
        """"balanced" or "splits" for decode rows that hold `kv_lens` tokens (host values; None: unknown). Equal cuts
        are a little faster while rows are alike (no walk crosses a row's end, one table read less before the first
        tile); one long row among short ones is where they lose: measured at 32 kv-head-8 rows, one of 8,192 tokens
        and 31 of 500, 36 µs against 56 µs."""
        if self.decode_attention != "auto":
            return self.decode_attention
        if kv_lens is None or len(kv_lens) < 2:
            return "splits"
        longest, total = int(max(kv_lens)), int(sum(int(v) for v in kv_lens))
        return "balanced" if longest >= 4096 and longest * len(kv_lens) >= 8 * total else "splits"

    def _split_cost(self, rows: int, heads: int, kv_heads: int, max_kv: int, splits: int) -> int:
        """Waves x (tiles a CTA walks + 1 for its start): what a launch of `splits` parts a row costs, in tile times."""
        ctas, tiles, slots = rows * kv_heads * (-(-(heads // kv_heads) // 16)), -(-max_kv // 64), 3 * self.sms
        return -(-ctas * splits // slots) * (-(-tiles // splits) + 1)

    def decode_splits(self, rows: int, heads: int, kv_heads: int, max_kv: int, most: int = 64) -> int:
        """Parts the keys of a decode row are cut into. Three CTAs fit an SM; a launch of `ctas * parts` CTAs runs in
        waves of 3 x SMs, each CTA walking its share of the longest row's 64-key tiles plus a fixed start-up of
        about one tile. The number of parts (1 to `most`) with the least waves x (tiles + 1) wins. It is a function of
        the batch's size and the longest length only, as the reference plans its splits
        (plugins/holon_plugins/kernels/triton_attn/plugin.py:40-96)."""
        key = (rows, heads, kv_heads, -(-max_kv // 64), most)
        if key not in self._splits:
            tiles = key[3]
            self._splits[key] = min(range(1, max(1, min(most, tiles)) + 1),
                                    key=lambda s: (self._split_cost(rows, heads, kv_heads, max_kv, s), s))
        return self._splits[key]

    MERGE_KERNEL_TILES = 6                    # what the second kernel and its scratch cost, in 64-key tile times

    def decode_cluster_splits(self, rows: int, heads: int, kv_heads: int, head_dim: int, max_kv: int, splits: int) -> int:
        """The number of splits (2 to 16) that merge inside the kernel as one thread-block cluster per (row, kv head),
        or 0 where `splits` parts and the merge kernel are the better plan. A cluster is taken only while all of them
        run at once (over several waves clusters leave holes: at 64 rows 16.6 ms a step against 15.4 ms with the merge
        kernel; the runtime says how many clusters of each size fit, and from 12 CTAs a cluster that is fewer than
        the CTA slots suggest); of those sizes the one whose CTAs walk the fewest tiles wins. Measured at 8,192 keys
        and 8 kv heads of 128, that cluster against the best number of splits with the merge kernel: 1 row 20.5 µs
        (16 CTAs) / 21.4, 3 rows 27.7 (15) / 29.7, 6 rows 38.9 (8) / 44.0, 8 rows 49.2 (6) / 56.2, 16 rows 87.0 (3) /
        93.2, 24 rows 122.9 (2) / 138.2; from 32 rows on no size fits one wave."""
        if not self.decode_cluster:
            return 0
        key = ("cluster", rows, heads, kv_heads, head_dim, -(-max_kv // 64), splits)
        if key not in self._splits:
            pairs, tiles = rows * kv_heads * (-(-(heads // kv_heads) // 16)), -(-max_kv // 64)
            fitting = [s for s in range(2, min(16, tiles) + 1) if pairs <= self._cluster_capacity(head_dim, s)]
            best = min(fitting, key=lambda s: (-(-tiles // s), s), default=0)
            merged = self._split_cost(rows, heads, kv_heads, max_kv, splits) + self.MERGE_KERNEL_TILES
            self._splits[key] = best if best and -(-tiles // best) + 1 <= merged else 0
        return self._splits[key]

    def _cluster_capacity(self, head_dim: int, splits: int) -> int:
        key = ("capacity", -(-head_dim // 64) if head_dim <= 128 else 3, splits)
        if key not in self._splits:
            fn = self.lib.hb_attention_decode_cluster_capacity
            fn.restype = ctypes.c_int
            self._splits[key] = int(fn(int(head_dim), int(splits)))
        return self._splits[key]

    def _attention_generic(self, out, q, kv, block_table, rows, scale, window, sinks=None) -> None:
        t, heads, head_dim = q.shape
        self._call("hb_attention_generic", self._p(out), self._p(q), self._p(kv), _code(q),
                   self._i32(block_table, "block_table"), block_table.shape[1], self._i32(rows.row_slot, "row_slot"),
                   self._i32(rows.query_start, "query_start"), self._i32(rows.kv_len, "kv_len"), rows.n_rows, t,
                   heads, kv.shape[2], head_dim, kv.shape[0], kv.shape[3], ctypes.c_float(scale), int(window),
                   self._p(sinks))

    # ---- the residual sum and the next norm inside the product that ends a part (decode steps)
    def can_link(self, rows: int, hidden: int, norm) -> bool:
        """Whether a product of `rows` rows may add itself into the stream and leave `norm`'s rows unscaled for the
        next product: both run in the weight-streaming kernels, which take SKINNY_ROWS rows and, on clusters, MID_ROWS."""
        w = getattr(norm, "weight", None)
        most = self.MID_ROWS if self.mid else self.WIDE_ROWS if self.skinny32 else self.SKINNY_ROWS
        return self.fused_norm and 0 < rows <= most and hidden % 8 == 0 and w is not None \
            and w.tensor.dtype in (torch.bfloat16, torch.float32) and w.tensor.shape == (hidden,)

    def linear_link(self, h, x, weight, norm_weight, eps: float, offset: float):
        """h [m, n] (float32) += bfloat16(x · weightᵀ) and, returned as parts.base.Scaled, the new h times
        (norm_weight + offset) in bfloat16 with the partial sums of squares its RMSNorm still needs. None, with
        nothing done, where the kernel does not apply (another dtype, k no multiple of 8, more rows)."""
        from ..parts.base import Scaled
        m, k = x.shape
        n = weight.shape[0]
        wide = self._wide_takes(m, weight)
        if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or h.dtype != torch.float32 or k % 8 \
                or not (0 < m <= (self.MID_ROWS if self.mid else self.SKINNY_ROWS) or wide) or tuple(h.shape) != (m, n) \
                or weight.shape != (n, k):
            return None
        self._check(h, x, weight, norm_weight)
        y = torch.empty((m, n), dtype=torch.bfloat16, device=self.device)
        if wide:
            ss = torch.empty((-(-n // 16), self.WIDE_ROWS), dtype=torch.float32, device=self.device)
            self._call("hb_gemm_bf16_skinny32", self._p(y), 0, self._p(x), self._p(weight), m, n, k, 3, 0, self._p(h),
                       self._p(norm_weight), int(norm_weight.dtype == torch.float32), ctypes.c_float(offset), self._p(ss),
                       None, 0, ctypes.c_float(0.0), 0)
            return Scaled(y, ss, float(eps), n)
        if m > self.SKINNY_ROWS:
            self.mid_launches += 1
            ss = torch.empty((-(-n // 256), self.MID_ROWS), dtype=torch.float32, device=self.device)
            self._call("hb_gemm_bf16_mid", self._p(y), 0, self._p(x), self._p(weight), m, n, k, 3, 0, self._p(h),
                       self._p(norm_weight), int(norm_weight.dtype == torch.float32), ctypes.c_float(offset), self._p(ss),
                       None, 0, 0, ctypes.c_float(0.0), 0, int(self.mid_split))
            return Scaled(y, ss, float(eps), n)
        parts = -(-n // 16)
        ss = torch.empty((parts, 16), dtype=torch.float32, device=self.device)
        if self._chains(m, k, x, weight, y) and norm_weight.dtype in (torch.bfloat16, torch.float32):
            self._queue(w=weight, x=x, out=y, mode=3, n=n, h=h, next_weight=norm_weight, next_offset=offset, ss_out=ss)
            return Scaled(y, ss, float(eps), n)
        self._call("hb_gemm_bf16_skinny_linked", self._p(y), 0, self._p(x), self._p(weight), m, n, k, 3, 0, self._p(h),
                   self._p(norm_weight), int(norm_weight.dtype == torch.float32), ctypes.c_float(offset), self._p(ss),
                   None, 0, ctypes.c_float(0.0), 0)
        return Scaled(y, ss, float(eps), n)

    def linear_dyt(self, h, x, weight, post, pre):
        """h [m, n] (float32) += N_post(bfloat16(x · weightᵀ)) with N(y) = tanh(alpha y) w + b for a triple (alpha, w, b) of
        float32 tensors, in the epilogue of the product for the few rows of a decode step; returns N_pre of the new h
        (bfloat16 [m, n]; `pre` None: True). None, with nothing done, where the kernel does not apply (another dtype, k
        no multiple of 8, more than SKINNY_ROWS rows)."""
        m, k = x.shape
        n = weight.shape[0]
        if not self.fused_norm or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or h.dtype != torch.float32 \
                or k % 8 or not 0 < m <= self.SKINNY_ROWS or tuple(h.shape) != (m, n) or weight.shape != (n, k) \
                or (x.data_ptr() | weight.data_ptr()) % 16 or not x.is_contiguous():
            return None
        tensors = [t for triple in (post, pre) if triple is not None for t in triple]
        self._check(h, x, weight, *tensors)
        self._f32("linear_dyt", *tensors)
        if any(t.numel() != n for triple in (post, pre) if triple is not None for t in triple[1:]):
            raise KernelError("linear_dyt: the norms' weights and biases must be [n]")
        out = torch.empty((m, n), dtype=torch.bfloat16, device=self.device) if pre is not None else None
        b = pre or (None, None, None)
        self._call("hb_gemm_bf16_skinny_dyt", self._p(out), self._p(x), self._p(weight), m, n, k, self._p(h), self._p(post[0]),
                   self._p(post[1]), self._p(post[2]), self._p(b[0]), self._p(b[1]), self._p(b[2]))
        return out if out is not None else True

    def _scaled_product(self, out, x, weight, mode: int, inter: int) -> None:
        """A product whose x is parts.base.Scaled: the weight-streaming kernel applies the row scale to its sums."""
        y = x.y
        self._check(out, y, x.ss, weight)
        m, k = y.shape
        if m > self.MID_ROWS or k % 8 or y.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.shape[1] != k:
            raise KernelError("a product of unscaled rows takes up to MID_ROWS bfloat16 rows of a multiple of 8 columns")
        if self._wide_takes(m, weight, x.ss.shape[1]):
            return self._call("hb_gemm_bf16_skinny32", self._p(out), int(out.dtype == torch.float32), self._p(y),
                              self._p(weight), m, weight.shape[0], k, mode, inter, None, None, 0, ctypes.c_float(0.0), None,
                              self._p(x.ss), x.ss.shape[0], ctypes.c_float(x.eps), x.dim)
        if m > self.SKINNY_ROWS or self._mid_takes(m, weight, mode):
            self.mid_launches += 1
            return self._call("hb_gemm_bf16_mid", self._p(out), int(out.dtype == torch.float32), self._p(y), self._p(weight),
                              m, weight.shape[0], k, mode, inter, None, None, 0, ctypes.c_float(0.0), None, self._p(x.ss),
                              x.ss.shape[0], x.ss.shape[1], ctypes.c_float(x.eps), x.dim, int(self.mid_split))
        if self._chains(m, k, y, weight) and out.dtype in (torch.bfloat16, torch.float32) and (mode == 0 or out.dtype == torch.bfloat16):
            self._queue(w=weight, x=x, out=out, mode=mode, n=weight.shape[0], inter=inter, scaled=x)
            return
        self._call("hb_gemm_bf16_skinny_linked", self._p(out), int(out.dtype == torch.float32), self._p(y), self._p(weight),
                   m, weight.shape[0], k, mode, inter, None, None, 0, ctypes.c_float(0.0), None, self._p(x.ss),
                   x.ss.shape[0], ctypes.c_float(x.eps), x.dim)

    def linear(self, out, x, weight) -> None:
        if hasattr(x, "ss"):                             # rows that lack their norm's scale (parts.base.Scaled)
            if weight.shape[1] != x.shape[1] or out.shape != (x.shape[0], weight.shape[0]):
                raise KernelError(f"linear: x {tuple(x.shape)} · w {tuple(weight.shape)}ᵀ -> out {tuple(out.shape)} do not fit")
            return self._scaled_product(out, x, weight, 0, 0)
        self._check(out, x, weight)
        m, k = x.shape
        n = weight.shape[0]
        if weight.shape != (n, k) or out.shape != (m, n) or x.dtype != weight.dtype:
            raise KernelError(f"linear: x {tuple(x.shape)} · w {tuple(weight.shape)}ᵀ -> out {tuple(out.shape)} do not fit")
        if self._pending:
            if self._chains(m, k, x, weight) and out.data_ptr() % 16 == 0 and self._pending[0][2] == m:
                self._queue(w=weight, x=x, out=out, mode=0, n=n)   # (the last of a run of products: with them, then out)
                return self.flush()
            self.flush()
        if x.dtype == torch.float32:
            if out.dtype != torch.float32:
                raise KernelError("linear: a float32 product writes float32")
            self._call("hb_gemm_f32", self._p(out), self._p(x), self._p(weight), m, n, k)
        elif m <= self.SKINNY_ROWS and k % 8 == 0:       # decode steps: bound by reading the weight once
            self._call("hb_gemm_bf16_skinny", self._p(out), int(out.dtype == torch.float32), self._p(x),
                       self._p(weight), m, n, k, 0, 0)
        elif self.gemm == "tcgen05" and k % 8 == 0:      # the hand-written tensor-memory kernel in place of the library
            self.linear_tcgen05(out, x, weight)
        elif out.dtype == torch.float32:                 # the head: bfloat16 operands, 32-bit logits
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        else:
            torch.mm(x, weight.t(), out=out)

    SKINNY_ROWS = 16
    MID_ROWS = 64                             # rows the clustered tcgen05 products take (csrc/gemm_mid.cu)

    def linear_mid(self, out, x, weight, swiglu: bool = False, split: int = 0) -> None:
        """The product (or SwiGLU's silu(gate) · up) of up to MID_ROWS bfloat16 rows on csrc/gemm_mid.cu, whatever the
        table's own choice for these sizes would be (tests, microbench); `split`: the cluster size (0: chosen)."""
        self._check(out, x, weight)
        m, k = x.shape
        n = weight.shape[0]
        inter = n // 2 if swiglu else 0
        if weight.shape != (n, k) or out.shape != (m, inter if swiglu else n) or x.dtype != torch.bfloat16 \
                or weight.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError("linear_mid: bfloat16 x [m, k] and w [n, k]; out [m, n] (or [m, n / 2]) bfloat16 or float32")
        self.mid_launches += 1
        self._call("hb_gemm_bf16_mid", self._p(out), int(out.dtype == torch.float32), self._p(x), self._p(weight), m, n, k,
                   int(swiglu), inter, None, None, 0, ctypes.c_float(0.0), None, None, 0, 0, ctypes.c_float(0.0), 0, int(split))

    def linear_tcgen05(self, out, x, weight, swiglu: bool = False, pair: bool | None = None) -> None:
        """The product (or, with `swiglu`, SwiGLU's silu(gate) · up) on the hand-written tcgen05 / TMA / TMEM kernels:
        `pair` picks the one that puts two CTAs on a 256 x 256 tile (default: self.gemm_pair)."""
        self._check(out, x, weight)
        m, k = x.shape
        n = weight.shape[0]
        inter = n // 2 if swiglu else 0
        if weight.shape != (n, k) or out.shape != (m, inter if swiglu else n) or x.dtype != torch.bfloat16 \
                or weight.dtype != torch.bfloat16 or out.dtype not in (torch.bfloat16, torch.float32):
            raise KernelError("linear_tcgen05: bfloat16 x [m, k] and w [n, k]; out [m, n] (or [m, n / 2]) bfloat16 or float32")
        name = "hb_gemm_bf16_tcgen05_pair" if (self.gemm_pair if pair is None else pair) else "hb_gemm_bf16_tcgen05"
        self._call(name, self._p(out), int(out.dtype == torch.float32), self._p(x), self._p(weight), m, n, k,
                   int(swiglu), inter)

    def status(self) -> int:
        """0, or the code of a bounded wait inside a kernel that gave up: (place << 28) | (block + 1). A read of host
        memory, no synchronisation: it tells of every kernel that has finished (wait for the step's event first)."""
        return int(self._status_word[0])

    def clear_status(self) -> None:
        self._status_word[0] = 0

    def status_selftest(self, polls: int = 1000) -> None:
        """Enqueues a wait of `polls` polls on a barrier nobody arrives at: it runs out and `status()` turns non-zero."""
        self._call("hb_status_selftest", int(polls))

    def tcgen05_status(self) -> int:
        """0, or which bounded wait inside a kernel (a tcgen05 product or attention, the chained products) gave up
        (synchronises the device; clears the kernels' words and the host's). After a wait of the chained products gave
        up their barrier and flags are put back to zero, so that the next launch starts clean."""
        out = 0
        for name in ("hb_gemm_tcgen05_status", "hb_gemm_tcgen05_pair_status", "hb_attention_tcgen05_status",
                     "hb_gemm_chain_status", "hb_gemm_tickets_status", "hb_gemm_mid_status", "hb_experts_tcgen05_status"):
            status = ctypes.c_uint(0)
            if getattr(self.lib, name)(ctypes.byref(status)):
                raise KernelError(self.lib.hb_last_error().decode())
            out = out or status.value
        self.clear_status()
        if out:
            self._chain_sync.zero_()
            self._chain_flags.zero_()
            self._ticket_state.zero_()
        return out

    def swiglu_gate_up(self, out, x, weight) -> None:
        """out [tokens, inter] = silu(x · gateᵀ) · (x · upᵀ) with gate's rows first in `weight` [2 inter, k]: for a
        few tokens one kernel with the activation in its epilogue, else the product and the activation kernel."""
        if hasattr(x, "ss"):                             # rows that lack their norm's scale (parts.base.Scaled)
            if weight.shape != (2 * out.shape[1], x.shape[1]) or out.shape[0] != x.shape[0] or out.dtype != torch.bfloat16:
                raise KernelError("swiglu_gate_up: x [tokens, k], weight [2 inter, k], out [tokens, inter], one dtype")
            return self._scaled_product(out, x, weight, 1, out.shape[1])
        self._check(out, x, weight)
        m, k = x.shape
        inter = out.shape[1]
        if weight.shape != (2 * inter, k) or out.shape[0] != m or not (out.dtype == x.dtype == weight.dtype):
            raise KernelError("swiglu_gate_up: x [tokens, k], weight [2 inter, k], out [tokens, inter], one dtype")
        if x.dtype == torch.bfloat16 and k % 8 == 0 and self._wide_takes(m, weight):
            return self._call("hb_gemm_bf16_skinny32", self._p(out), 0, self._p(x), self._p(weight), m, 2 * inter, k, 1, inter,
                              None, None, 0, ctypes.c_float(0.0), None, None, 0, ctypes.c_float(0.0), 0)
        if x.dtype == torch.bfloat16 and k % 8 == 0 and self._mid_takes(m, weight, 1):
            return self.linear_mid(out, x, weight, swiglu=True, split=self.mid_split)
        if x.dtype == torch.bfloat16 and m <= self.SKINNY_ROWS and k % 8 == 0:
            self._call("hb_gemm_bf16_skinny", self._p(out), 0, self._p(x), self._p(weight), m, 2 * inter, k, 1, inter)
            return
        if x.dtype == torch.bfloat16 and k % 8 == 0 and self.gemm != "cublas":
            # Measured at 24576 x 4096 against the library's product plus the activation kernel: by CTA pairs 66 us
            # against 74 at 256 rows, 280 against 317 at 2,048, 555 against 627 at 4,096, but 1,226 against 1,202 at
            # 8,192; one CTA a tile 59 against 66 at 128 rows; below about 100 rows the library wins (64 against 70).
            if self.gemm == "tcgen05" or 192 < m <= 6144:
                self.linear_tcgen05(out, x, weight, swiglu=True)
                return
            if 96 < m <= 192:
                self.linear_tcgen05(out, x, weight, swiglu=True, pair=False)
                return
        gate_up = torch.empty(m, 2 * inter, dtype=x.dtype, device=self.device)
        self.linear(gate_up, x, weight)
        self.silu_mul(out, gate_up)

    # ------------------------------------------------------------------ hyper-connections, latent attention, experts
    def hyper_mix_norm(self, out, xs, src, y, mix, outc, inc, weight, eps, offset, index) -> None:
        self._check(out, xs, src, y, mix, outc, inc, weight, index)
        t, streams, dim = xs.shape
        rows = index.shape[0] if index is not None else t
        if xs.dtype != torch.float32 or out.shape != (rows, dim) or weight.shape != (dim,):
            raise KernelError("hyper_mix_norm: xs float32 [tokens, streams, dim], out [rows, dim], weight [dim]")
        if (src is not None and (src.dtype != torch.float32 or src.shape != (t, dim))) \
                or (y is not None and (y.shape != (t, dim) or y.dtype != out.dtype)):
            raise KernelError("hyper_mix_norm: src float32 [tokens, dim], y [tokens, dim] of out's dtype")
        for name, c, shape in (("mix", mix, (streams, streams)), ("out", outc, (streams,)), ("in", inc, (streams,))):
            if c is not None and (c.dtype != torch.float32 or c.shape != shape):
                raise KernelError(f"hyper_mix_norm: {name} must be float32 {shape}")
        self._call("hb_hyper_mix_norm", self._p(out), _code(out), self._p(xs), self._p(src), self._p(y), self._p(mix),
                   self._p(outc), self._p(inc), self._p(weight), _code(weight), ctypes.c_float(eps), ctypes.c_float(offset),
                   self._i32(index, "index"), rows, dim, streams)

    def latent_prepare(self, qa, first, heads, dim, rot, rank, dkv_at, positions, table, rot_dims, norm_weight, eps,
                       cache, write_index) -> None:
        self._check(qa, first, positions, table, norm_weight, cache, write_index)
        t, ld = first.shape
        if qa.shape != (t, heads, rank + rot) or qa.dtype != first.dtype or ld < heads * (dim + rot):
            raise KernelError("latent_prepare: first [tokens, >= heads (dim + rot)], qa [tokens, heads, rank + rot], one dtype")
        if table is not None and (table.dtype != torch.float32 or table.shape[1] != rot_dims):
            raise KernelError("latent_prepare: the rotation table must be float32 [positions, rot_dims]")
        if cache is not None and (cache.dtype != first.dtype or cache.dim() != 3 or cache.shape[2] != rank + rot):
            raise KernelError("latent_prepare: cache must be [pages, page_size, rank + rot] of first's dtype")
        self._call("hb_latent_prepare", self._p(qa), self._p(first), _code(first), ld, t, heads, dim, rot, rank, int(dkv_at),
                   self._i32(positions, "positions"), self._p(table), int(rot_dims), table.shape[0] if table is not None else 0,
                   self._p(norm_weight), _code(norm_weight) if norm_weight is not None else 0, ctypes.c_float(eps),
                   self._p(cache), self._i32(write_index, "write_index"), cache.shape[0] if cache is not None else 0,
                   cache.shape[1] if cache is not None else 1)

    def linear_heads(self, out, x, w) -> None:
        """out[t, b, :] = x[t, b, :] · w[b]ᵀ for every head b: x [tokens, heads, k] and out [tokens, heads, n] may be
        views into wider rows (innermost stride 1), w [heads, n, k] contiguous. float32: the library's own kernel with
        a fixed summation order; bfloat16: one batched product of cuBLAS through torch, as `linear` uses it."""
        self._check(w)
        t, b, k = x.shape
        n = w.shape[1]
        if w.shape != (b, n, k) or out.shape != (t, b, n) or not (out.dtype == x.dtype == w.dtype) \
                or x.stride(2) != 1 or out.stride(2) != 1 or x.get_device() != self._index or out.get_device() != self._index:
            raise KernelError(f"linear_heads: x {tuple(x.shape)} · w {tuple(w.shape)}ᵀ -> out {tuple(out.shape)} do not fit")
        if t == 0:
            return
        if x.dtype == torch.float32:
            self._call("hb_gemm_f32_heads", self._p(out), self._p(x), self._p(w), t, n, k, b,
                       ctypes.c_long(x.stride(0)), ctypes.c_long(x.stride(1)), ctypes.c_long(out.stride(0)),
                       ctypes.c_long(out.stride(1)))
        else:
            if self._pending:
                self.flush()
            torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))

    def latent_attention(self, out, qa, cache, block_table, rows, scale, rank, window) -> None:
        self._check(out, qa, cache, block_table, rows.row_slot, rows.query_start, rows.kv_len)
        t, heads, dk = qa.shape
        if out.shape != (t, heads, rank) or cache.dim() != 3 or cache.shape[2] != dk or not (out.dtype == qa.dtype == cache.dtype):
            raise KernelError("latent_attention: qa [tokens, heads, rank + rot], out [tokens, heads, rank], cache [pages, "
                              "page_size, rank + rot], one dtype")
        rot = dk - rank
        common = (self._i32(block_table, "block_table"), block_table.shape[1], self._i32(rows.row_slot, "row_slot"),
                  self._i32(rows.query_start, "query_start"), self._i32(rows.kv_len, "kv_len"))
        fast = qa.dtype == torch.bfloat16 and rank % 16 == 0 and rot % 16 == 0 and 16 <= rank <= 512 \
            and self.attention_bf16 == "fast"
        if not fast:                                  # float32, and sizes the tensor-core kernel does not take
            return self._call("hb_latent_attention_generic", self._p(out), self._p(qa), self._p(cache), _code(qa), *common,
                              rows.n_rows, t, heads, rank, rot, cache.shape[0], cache.shape[1], ctypes.c_float(scale),
                              int(window))
        sizes = (heads, rank, rot, cache.shape[0], cache.shape[1], ctypes.c_float(scale), int(window))
        ones = rows.n_decode
        if ones:                                      # rows of one token: their keys cut into parts that fill the GPU
            splits = self.latent_splits(ones, heads, rank, rows.max_kv)
            scratch = torch.empty(ones * heads * splits * (rank + 2), dtype=torch.float32, device=self.device) \
                if splits > 1 else None
            self._call("hb_latent_attention_bf16", self._p(out), self._p(scratch), self._p(qa), self._p(cache), *common,
                       0, ones, 0, ones, *sizes, splits)
        if rows.n_rows > ones:
            self._call("hb_latent_attention_bf16", self._p(out), None, self._p(qa), self._p(cache), *common, ones,
                       rows.n_rows, ones, t - ones, *sizes, 1)

    def latent_splits(self, rows: int, heads: int, rank: int, max_kv: int) -> int:
        """Parts the keys of one-token rows are cut into for the latent attention kernel: enough that two CTAs an SM
        have work, each part at least one tile of 64 keys, at most 32. A function of the batch's size and the longest
        row only (under a CUDA graph: of the bucket its plan pinned)."""
        if self.latent_split:                                            # (tests: a fixed number of parts)
            return int(self.latent_split)
        tile = 64 if rank <= 128 else 32 if rank <= 256 else 16          # (token, head) pairs a CTA of four warps
        ctas = rows * (-(-heads // tile))
        return max(1, min(32, -(-max_kv // 64), (2 * self.sms) // max(1, ctas)))

    def sigmoid_gate(self, o, g) -> None:
        """o [tokens, n] *= sigmoid(g [tokens, n]); g may be a view into wider rows."""
        self._check(o)
        if g.shape != o.shape or g.dtype != o.dtype or g.stride(1) != 1 or g.get_device() != self._index:
            raise KernelError("sigmoid_gate: g must have o's shape and dtype, innermost stride 1")
        self._call("hb_sigmoid_gate", self._p(o), self._p(g), _code(o), o.shape[0], o.shape[1], ctypes.c_long(g.stride(0)))

    def activation(self, x, act: int, numbers=None) -> None:
        """x = act(x) in place; `numbers` (float32 [2]) for act 4 (xielu)."""
        self._check(x, numbers)
        self._f32("activation", numbers)
        if numbers is not None and numbers.numel() != 2:
            raise KernelError("activation: xielu takes two numbers")
        self._call("hb_activation", self._p(x), _code(x), ctypes.c_long(x.numel()), int(act), self._p(numbers))

    def route_top(self, chosen, weight, counts, z, experts, scale, renormalize, bias=None, correction=None, groups=1,
                  keep=1, tiny=0.0) -> None:
        """`bias` (float32 [experts] or None) is added to the logits before anything else. `correction` (float32 [experts]
        or None) is added to the softmax scores for the choice alone; `groups` > 1: experts in that many equal groups of
        neighbours, of which the `keep` best (by their best choice score) stay in the running; `tiny` is added to the
        chosen scores' sum before `renormalize` divides."""
        self._check(chosen, weight, counts, z, bias, correction)
        self._f32("route_top", bias, correction)
        t, top = chosen.shape
        if z.dtype != torch.float32 or z.shape[0] != t or z.shape[1] < experts or weight.shape != (t, top) \
                or weight.dtype != torch.float32 or counts.shape[0] < 2 * experts + 1:
            raise KernelError("route_top: z float32 [tokens, >= experts], chosen int32 and weight float32 [tokens, top], "
                              "counts int32 [2 experts + 1]")
        self._call("hb_route_top", self._i32(chosen, "chosen"), self._p(weight), self._i32(counts, "counts"), self._p(z),
                   self._p(bias), z.shape[1], t, int(experts), top, ctypes.c_float(scale), int(bool(renormalize)),
                   self._p(correction), int(groups), int(keep), ctypes.c_float(tiny))

    def route_rows(self, chosen, weight, counts, place, token_of, z, experts, scale, renormalize, bias=None,
                   correction=None, groups=1, keep=1, tiny=0.0) -> None:
        """`route_top` and `expert_rows` as one call (one launch for a few tokens). counts int32 [2 experts + 3] need not
        be zeroed; afterwards counts[2 experts + 1:] = (0, tokens)."""
        self._check(chosen, weight, counts, place, token_of, z, bias, correction)
        self._f32("route_rows", bias, correction)
        if correction is not None and correction.shape != (experts,):
            raise KernelError("route_rows: correction must be float32 [experts]")
        t, top = chosen.shape
        if z.dtype != torch.float32 or z.shape[0] != t or z.shape[1] < experts or weight.shape != (t, top) \
                or weight.dtype != torch.float32 or counts.shape[0] < 2 * experts + 3 or place.shape[0] != t * top \
                or token_of.shape[0] != t * top:
            raise KernelError("route_rows: z float32 [tokens, >= experts], chosen int32 and weight float32 [tokens, top], "
                              "counts int32 [2 experts + 3], place and token_of int32 [tokens * top]")
        self._call("hb_route_rows", self._i32(chosen, "chosen"), self._p(weight), self._i32(counts, "counts"),
                   self._i32(place, "place"), self._i32(token_of, "token_of"), self._p(z), self._p(bias), z.shape[1], t, int(experts), top,
                   ctypes.c_float(scale), int(bool(renormalize)), self._p(correction), int(groups), int(keep), ctypes.c_float(tiny))

    def expert_rows(self, place, token_of, counts, chosen, experts) -> None:
        self._check(place, token_of, counts, chosen)
        t, top = chosen.shape
        if place.shape[0] != t * top or token_of.shape[0] != t * top or counts.shape[0] < 2 * experts + 1:
            raise KernelError("expert_rows: place and token_of int32 [tokens * top], counts int32 [2 experts + 1]")
        self._call("hb_expert_rows", self._i32(place, "place"), self._i32(token_of, "token_of"), self._i32(counts, "counts"),
                   self._i32(chosen, "chosen"), t, top, int(experts))

    EXPERT_TCGEN05_ROWS = 96                  # rows an expert on average from which its products run on tcgen05

    def expert_linear(self, out, x, token_of, w, starts, act: int) -> None:
        self._check(out, x, token_of, w, starts)
        e, n, k = w.shape
        rows = out.shape[0]
        if out.shape != (rows, n) or x.shape[1] != k or not (out.dtype == x.dtype == w.dtype) or starts.shape[0] != e + 1 \
                or (token_of is None and x.shape[0] != rows) or (token_of is not None and token_of.shape[0] != rows):
            raise KernelError("expert_linear: x [*, k], w [experts, n, k], out [rows, n], starts int32 [experts + 1]")
        aligned = k % 8 == 0 and n % 8 == 0 and (x.data_ptr() | w.data_ptr() | out.data_ptr()) % 16 == 0
        if x.dtype == torch.bfloat16 and aligned and (self.expert_products == "tcgen05" or (
                self.expert_products == "fast" and self.expert_tile_rows == 0 and rows >= self.EXPERT_TCGEN05_ROWS * e)):
            # prompts (a hundred rows an expert and more): the tcgen05 kernel, x gathered expert by expert first
            tiles = -(-rows // 128) + min(e, rows)
            table = torch.empty(3 * tiles, dtype=torch.int32, device=self.device)
            gathered = torch.empty((rows, k), dtype=x.dtype, device=self.device) if token_of is not None else None
            return self._call("hb_expert_linear_tcgen05", self._p(out), self._p(x), self._i32(token_of, "token_of"),
                              self._p(gathered), self._p(w), self._i32(starts, "starts"), self._i32(table, "table"), rows, e, n, k,
                              int(act))
        if x.dtype == torch.bfloat16 and aligned and self.expert_products in ("fast", "mma"):
            return self._call("hb_expert_linear_bf16", self._p(out), self._p(x), self._i32(token_of, "token_of"), self._p(w),
                              self._i32(starts, "starts"), rows, e, n, k, int(act), int(self.expert_tile_rows))
        self._call("hb_expert_linear", self._p(out), self._p(x), _code(x), self._i32(token_of, "token_of"), self._p(w),
                   self._i32(starts, "starts"), rows, e, n, k, int(act))

    def expert_combine(self, out, y, place, weight, shared, z, experts, x=None, identity_from=None) -> None:
        """`z` None with `shared`: the shared rows are added without a gate. `x` [tokens, hidden] and `identity_from`
        (int32 [1] on the device): pairs whose row is identity_from[0] or later read x[token] in place of y."""
        self._check(out, y, place, weight, shared, z, x, identity_from)
        t, hidden = out.shape
        top = weight.shape[1]
        if y.shape != (t * top, hidden) or y.dtype != out.dtype or place.shape[0] != t * top \
                or (shared is not None and (shared.shape != out.shape or shared.dtype != out.dtype))\
                or (z is not None and (z.dtype != torch.float32 or z.shape[1] <= experts)) \
                or (x is None) != (identity_from is None) or (x is not None and (x.shape != out.shape or x.dtype != out.dtype)):
            raise KernelError("expert_combine: y [tokens * top, hidden], shared and x [tokens, hidden], z float32 [tokens, > experts]")
        self._call("hb_expert_combine", self._p(out), self._p(y), _code(out), self._i32(place, "place"), self._p(weight),
                   self._p(shared), self._p(z), z.shape[1] if z is not None else 0, int(experts), t, top, hidden,
                   self._p(x), self._i32(identity_from, "identity_from"))

    # ---- a block whose parts run side by side, an embedding with a pair table, mixers with a matrix state per head
    def embed_pair(self, out, table, scale, pair, ids, positions, rows, prev, mul_prev, mul_cur, buckets) -> None:
        """out = table[ids] · scale + pair[row of (previous id, id)] (csrc/api.h: hb_embed_pair); `prev` int32 [slots]."""
        self._check(out, table, pair, ids, positions, rows.query_start, rows.row_slot, prev)
        if out.dtype != torch.float32 or out.shape != (ids.shape[0], table.shape[1]):
            raise KernelError("embed_pair: out must be float32 [tokens, hidden]")
        if pair is not None and (pair.dtype != table.dtype or pair.shape != (buckets + 1, table.shape[1])):
            raise KernelError("embed_pair: the pair table must be [buckets + 1, hidden] of the table's dtype")
        self._call("hb_embed_pair", self._p(out), self._p(table), _code(table), ctypes.c_float(scale), self._p(pair),
                   self._i32(ids, "ids"), self._i32(positions, "positions"), self._i32(rows.query_start, "query_start"),
                   self._i32(rows.row_slot, "row_slot"), self._i32(prev, "prev"), rows.n_rows, ids.shape[0],
                   table.shape[1], table.shape[0], ctypes.c_long(mul_prev), ctypes.c_long(mul_cur), int(buckets))

    def sum_into(self, h, terms, bias=None) -> None:
        """h (float32 [tokens, hidden]) += Σ scale · x over `terms` [(x, scale), ...] (up to four) + bias."""
        xs = [x for x, _ in terms]
        self._check(h, bias, *xs)
        if not 1 <= len(terms) <= 4 or h.dtype != torch.float32 or any(x.shape != h.shape or x.dtype != xs[0].dtype for x in xs):
            raise KernelError("sum_into: one to four terms of h's shape and one dtype, h float32")
        if bias is not None and (bias.shape != (h.shape[1],) or bias.dtype != xs[0].dtype):
            raise KernelError("sum_into: bias must be [hidden] of the terms' dtype")
        xs += [None] * (4 - len(xs))
        scales = [float(sc) for _, sc in terms] + [0.0] * (4 - len(terms))
        self._call("hb_sum_into", self._p(h), *(self._p(x) for x in xs), *(ctypes.c_float(sc) for sc in scales),
                   self._p(bias), _code(terms[0][0]), h.shape[0], h.shape[1])

    def sum_norm(self, h, terms, bias, out, weight, eps, offset) -> None:
        """`sum_into`, and out = RMSNorm(h) · (weight + offset) of the summed rows, in one kernel."""
        xs = [x for x, _ in terms]
        self._check(h, bias, out, weight, *xs)
        if not 1 <= len(terms) <= 4 or h.dtype != torch.float32 or any(x.shape != h.shape or x.dtype != xs[0].dtype for x in xs) \
                or out.shape != h.shape or out.dtype != xs[0].dtype or weight.shape != (h.shape[1],):
            raise KernelError("sum_norm: one to four terms and out of h's shape and one dtype, h float32, weight [hidden]")
        if bias is not None and (bias.shape != (h.shape[1],) or bias.dtype != xs[0].dtype):
            raise KernelError("sum_norm: bias must be [hidden] of the terms' dtype")
        xs += [None] * (4 - len(xs))
        scales = [float(sc) for _, sc in terms] + [0.0] * (4 - len(terms))
        self._call("hb_sum_norm", self._p(h), *(self._p(x) for x in xs), *(ctypes.c_float(sc) for sc in scales),
                   self._p(bias), _code(out), self._p(out), self._p(weight), _code(weight), ctypes.c_float(eps),
                   ctypes.c_float(offset), h.shape[0], h.shape[1])

    def glu_clamped(self, out, gate_up, bias, limit, alpha) -> None:
        self._check(out, gate_up, bias)
        if gate_up.shape != (out.shape[0], 2 * out.shape[1]) or out.dtype != gate_up.dtype \
                or (bias is not None and (bias.shape != (gate_up.shape[1],) or bias.dtype != out.dtype)):
            raise KernelError("glu_clamped: gate_up [tokens, 2 inter] and bias [2 inter] of out's dtype")
        self._call("hb_glu_clamped", self._p(out), self._p(gate_up), self._p(bias), _code(out), ctypes.c_float(limit),
                   ctypes.c_float(alpha), out.shape[0], out.shape[1])

    @staticmethod
    def _f32(what: str, *tensors) -> None:
        for t in tensors:
            if t is not None and t.dtype != torch.float32:
                raise KernelError(f"{what}: 32-bit tensors expected, got {t.dtype}")

    def recurrent_scan(self, out, qk, v, decay, head_decay, beta, state, rows, token_decay=None, rate=None) -> None:
        """The token-by-token update of a matrix state per head (csrc/api.h: hb_recurrent_scan). `rate` (float32 [tokens,
        heads, dim], with `decay`, without `beta`): the generalized delta rule, S ← diag(decay) S − (rate ∘ k)(kᵀ S) + k vᵀ."""
        self._check(out, qk, v, decay, head_decay, beta, state, rows.query_start, rows.row_slot, token_decay, rate)
        self._f32("recurrent_scan", out, qk, v, decay, head_decay, beta, state, token_decay, rate)
        if rate is not None and (decay is None or rate.shape != decay.shape):
            raise KernelError("recurrent_scan: rate goes with decay and has its shape")
        t, heads, vdim = v.shape
        kv_heads, dim = qk.shape[2], qk.shape[3]
        if qk.shape != (t, 2, kv_heads, dim) or out.shape != v.shape or state.shape[1:] != (heads, vdim, dim) \
                or (decay is not None and decay.shape != (t, heads, dim)) or (beta is not None and beta.shape != (t, heads)) \
                or (head_decay is not None and head_decay.shape != (heads,)) \
                or (token_decay is not None and token_decay.shape != (t, heads)):
            raise KernelError("recurrent_scan: qk [tokens, 2, kv_heads, dim], v and out [tokens, heads, vdim], state "
                              "[slots, heads, vdim, dim], decay [tokens, heads, dim] or head_decay [heads], beta [tokens, heads]")
        self._call("hb_recurrent_scan", self._p(out), self._p(qk), self._p(v), self._p(decay), self._p(head_decay),
                   self._p(token_decay), self._p(beta), self._p(rate), self._p(state), self._i32(rows.query_start, "query_start"),
                   self._i32(rows.row_slot, "row_slot"), rows.n_rows, heads, kv_heads, dim, vdim,
                   int(getattr(rows, "max_q", 0) or 0))

    def delta_prepare(self, qk, v, beta, decay, gate, first, conv, conv_state, low2, dt_bias, rate_log, rows, q_scale,
                      unit_eps) -> None:
        """From a delta-rule mixer's first product and its low-rank projections' outputs to the scan's inputs
        (csrc/api.h: hb_delta_prepare)."""
        self._check(qk, v, beta, decay, gate, first, conv, conv_state, low2, dt_bias, rate_log, rows.query_start, rows.row_slot)
        self._f32("delta_prepare", qk, v, beta, decay, gate, low2, dt_bias, rate_log)
        t, heads, vdim = v.shape
        kv_heads, dim = qk.shape[2], qk.shape[3]
        taps = conv.shape[1]
        channels = 2 * kv_heads * dim + heads * vdim
        if first.shape != (t, channels + heads) or conv.shape[0] != channels or conv.dtype != first.dtype \
                or low2.shape != (t, heads * dim + heads * vdim) \
                or (taps > 1 and (conv_state is None or conv_state.shape[1:] != (taps - 1, channels) or conv_state.dtype != first.dtype)):
            raise KernelError("delta_prepare: first [tokens, q | k | v | b], conv [channels, taps], conv_state [slots, "
                              "taps - 1, channels] of one dtype, low2 float32 [tokens, heads dim + heads vdim]")
        self._call("hb_delta_prepare", self._p(qk), self._p(v), self._p(beta), self._p(decay), self._p(gate),
                   self._p(first), _code(first), first.shape[1], self._p(conv), taps, self._p(conv_state), self._p(low2),
                   self._p(dt_bias), self._p(rate_log), self._i32(rows.query_start, "query_start"),
                   self._i32(rows.row_slot, "row_slot"), rows.n_rows, t, heads, kv_heads, dim, vdim,
                   ctypes.c_float(q_scale), ctypes.c_float(unit_eps))

    def conv_carry(self, conv_state, first, channels, taps, rows) -> None:
        if taps <= 1:
            return
        self._check(conv_state, first, rows.query_start, rows.row_slot)
        self._call("hb_conv_carry", self._p(conv_state), self._p(first), _code(first), first.shape[1], channels, taps,
                   self._i32(rows.query_start, "query_start"), self._i32(rows.row_slot, "row_slot"), rows.n_rows)

    def retention_prepare(self, qk, v, first, positions, table, rot_dims, k_scale) -> None:
        self._check(qk, v, first, positions, table)
        self._f32("retention_prepare", qk, v, table)
        t, heads, vdim = v.shape
        dim = qk.shape[3]
        if qk.shape != (t, 2, heads, dim) or first.shape[0] != t or first.shape[1] < 2 * heads * dim + heads * vdim \
                or (rot_dims and (table is None or table.shape[1] != rot_dims)):
            raise KernelError("retention_prepare: qk [tokens, 2, heads, dim], v [tokens, heads, vdim], first [tokens, q | k | v | ...]")
        self._call("hb_retention_prepare", self._p(qk), self._p(v), self._p(first), _code(first), first.shape[1],
                   self._i32(positions, "positions"), self._p(table), int(rot_dims),
                   table.shape[0] if table is not None else 0, t, heads, dim, vdim, ctypes.c_float(k_scale))

    def gdelta_prepare(self, qk, v, decay, rate, first, pre, decay_bias, rate_bias, decay_scale, unit_eps) -> None:
        """From the generalized delta rule's first product [tokens, r | k | v | g | a] and its low-rank decay projection's
        output `pre` (float32 [tokens, heads dim]) to the scan's inputs (csrc/api.h: hb_gdelta_prepare)."""
        self._check(qk, v, decay, rate, first, pre, decay_bias, rate_bias)
        self._f32("gdelta_prepare", qk, v, decay, rate, pre, decay_bias, rate_bias)
        t, heads, dim = v.shape
        n = heads * dim
        if qk.shape != (t, 2, heads, dim) or decay.shape != v.shape or rate.shape != v.shape or first.shape[0] != t \
                or first.shape[1] < 5 * n or pre.shape != (t, n) or decay_bias.shape != (n,) or rate_bias.shape != (n,):
            raise KernelError("gdelta_prepare: first [tokens, >= 5 heads dim], pre [tokens, heads dim], qk [tokens, 2, heads, "
                              "dim], v, decay and rate [tokens, heads, dim], biases [heads dim]")
        self._call("hb_gdelta_prepare", self._p(qk), self._p(v), self._p(decay), self._p(rate), self._p(first), _code(first),
                   ctypes.c_long(first.shape[1]), self._p(pre), self._p(decay_bias), self._p(rate_bias), t, heads, dim,
                   ctypes.c_float(decay_scale), ctypes.c_float(unit_eps))

    def head_norm_gate(self, out, o, weight, gate_mul, gate_pre, eps, gate: str = "silu") -> None:
        """out = o / rms(o) · weight · gate per head; `gate_pre` may be a view into wider rows (silu of it is the gate, or
        with `gate="sigmoid"` its sigmoid); `weight` [vdim] for all heads or [heads vdim]."""
        if gate not in ("silu", "sigmoid"):
            raise KernelError(f"head_norm_gate: gate {gate!r}; known: silu, sigmoid")
        self._check(out, o, weight, gate_mul)
        self._f32("head_norm_gate", o, weight, gate_mul)
        t, heads, vdim = o.shape
        ld = 0
        if gate_pre is not None:
            if gate_pre.shape != (t, heads * vdim) or gate_pre.dtype != out.dtype or gate_pre.stride(1) != 1 \
                    or gate_pre.get_device() != self._index:
                raise KernelError("head_norm_gate: gate_pre must be [tokens, heads vdim] of out's dtype, innermost stride 1")
            ld = gate_pre.stride(0)
        per_head = weight is not None and heads > 1 and weight.shape == (heads * vdim,)
        if out.shape != o.shape or (weight is not None and weight.shape != (vdim,) and not per_head) \
                or (gate_mul is not None and gate_mul.numel() != o.numel()):
            raise KernelError("head_norm_gate: out and o [tokens, heads, vdim], weight [vdim] or [heads vdim], gate_mul of o's size")
        self._call("hb_head_norm_gate", self._p(out), self._p(o), _code(out), self._p(weight), self._p(gate_mul),
                   self._p(gate_pre), ctypes.c_long(ld), ctypes.c_float(eps), t, heads, vdim, int(per_head),
                   int(gate == "sigmoid"))

    # ---- a norm without statistics and the blend with the token before (csrc/dyt.cu)
    def dyt_add_norm(self, h, y, post, out, pre, index) -> None:
        """With N(x) = tanh(alpha x) w + b for a triple (alpha, w, b) of float32 tensors: h (float32 [tokens, dim]) +=
        N_post(y) (`post` None: y as it is; `y` None: nothing is added); out = N_pre of the sums, of all rows or of the
        rows `index` (then h stays as it is). `h` None: out = N_pre(y), rows of any number of dimensions."""
        tensors = [t for triple in (post, pre) if triple is not None for t in triple]
        self._check(h, y, out, index, *tensors)
        self._f32("dyt_add_norm", h, *tensors)
        src = h if h is not None else y
        dim = src.shape[-1]
        rows = index.shape[0] if index is not None else src.numel() // dim
        if (h is not None and y is not None and y.shape != h.shape) or (out is not None and (pre is None or out.numel() != rows * dim)) \
                or any(t.numel() != dim for triple in (post, pre) if triple is not None for t in triple[1:]):
            raise KernelError("dyt_add_norm: h and y [tokens, dim], out [rows, dim], weights and biases [dim]")
        a, b = post or (None, None, None), pre or (None, None, None)
        self._call("hb_dyt_add_norm", self._p(h), self._p(y), _code(y) if y is not None else 0, self._p(a[0]), self._p(a[1]),
                   self._p(a[2]), self._p(out), _code(out) if out is not None else 0, self._p(b[0]), self._p(b[1]), self._p(b[2]),
                   self._i32(index, "index"), rows, dim)

    def dyt_shift(self, out, into, h, y, post, pre, mix, carried, rows) -> None:
        """x = h + N_post(y) goes to `into` (h itself where y is None); n = N_pre(x); out_t = n_t + (n_(t-1) − n_t) · mix,
        the first token of a row reading n_(t-1) from carried[slot] (float32 [slots, dim]), which then receives the row's
        last n (csrc/api.h: hb_dyt_shift)."""
        tensors = [t for triple in (post, pre) if triple is not None for t in triple]
        self._check(out, into, h, y, mix, carried, rows.query_start, rows.row_slot, *tensors)
        self._f32("dyt_shift", into, h, mix, carried, *tensors)
        t, dim = h.shape
        if out.shape != h.shape or into.shape != h.shape or (y is not None and (y.shape != h.shape or into is h)) \
                or mix.shape != (dim,) or carried.shape[1:] != (dim,) or pre is None:
            raise KernelError("dyt_shift: out, into, h, y [tokens, dim] (into apart from h with y), mix [dim], carried [slots, dim]")
        a = post or (None, None, None)
        self._call("hb_dyt_shift", self._p(out), _code(out), self._p(into), self._p(h), self._p(y),
                   _code(y) if y is not None else 0, self._p(a[0]), self._p(a[1]), self._p(a[2]), self._p(pre[0]),
                   self._p(pre[1]), self._p(pre[2]), self._p(mix), self._p(carried), self._i32(rows.query_start, "query_start"),
                   self._i32(rows.row_slot, "row_slot"), rows.n_rows, t, dim)

    # ---- the matrix memory with exponential gates (csrc/mlstm.cu)
    def mlstm_gates(self, out, pre, bias, cap, m_state, rows) -> None:
        """out float32 [3, tokens, heads] = keep, take, exp(-m) from the gates' pre-activations `pre` float32 [tokens, >= 2
        heads] (input gates, then forget gates), bias [2 heads]; m_state float32 [slots, heads] carries the maximum."""
        self._check(out, pre, bias, m_state, rows.query_start, rows.row_slot)
        self._f32("mlstm_gates", out, pre, m_state)
        _, t, heads = out.shape
        if out.shape[0] != 3 or pre.shape[0] != t or pre.shape[1] < 2 * heads or m_state.shape[1:] != (heads,) \
                or (bias is not None and bias.shape != (2 * heads,)):
            raise KernelError("mlstm_gates: out [3, tokens, heads], pre [tokens, >= 2 heads], bias [2 heads], m_state [slots, heads]")
        self._call("hb_mlstm_gates", self._p(out), self._p(pre), pre.shape[1], self._p(bias),
                   _code(bias) if bias is not None else 0, ctypes.c_float(cap), self._p(m_state),
                   self._i32(rows.query_start, "query_start"), self._i32(rows.row_slot, "row_slot"), rows.n_rows, t, heads)

    def mlstm_prepare(self, qk, v1, take, first, q_scale) -> None:
        self._check(qk, v1, take, first)
        self._f32("mlstm_prepare", qk, v1, take)
        t, heads, vd1 = v1.shape
        dim = qk.shape[3]
        if qk.shape != (t, 2, heads, dim) or take.shape != (t, heads) or first.shape[0] != t \
                or first.shape[1] < 2 * heads * dim + heads * (vd1 - 1):
            raise KernelError("mlstm_prepare: qk [tokens, 2, heads, dim], v1 [tokens, heads, vdim + 1], take [tokens, heads], "
                              "first [tokens, q | k | v | ...]")
        self._call("hb_mlstm_prepare", self._p(qk), self._p(v1), self._p(take), self._p(first), _code(first), first.shape[1], t,
                   heads, dim, vd1 - 1, ctypes.c_float(q_scale))

    def mlstm_read_out(self, out, o1, floor, weight, gate_pre, eps, tiny) -> None:
        self._check(out, o1, floor, weight)
        self._f32("mlstm_read_out", o1, floor)
        t, heads, vdim = out.shape
        if o1.shape != (t, heads, vdim + 1) or floor.shape != (t, heads) or weight.shape != (heads * vdim,) \
                or gate_pre.shape != (t, heads * vdim) or gate_pre.dtype != out.dtype or gate_pre.stride(1) != 1 \
                or gate_pre.get_device() != self._index:
            raise KernelError("mlstm_read_out: out [tokens, heads, vdim], o1 [tokens, heads, vdim + 1], floor [tokens, heads], "
                              "weight [heads vdim], gate_pre [tokens, heads vdim] of out's dtype, innermost stride 1")
        self._call("hb_mlstm_read_out", self._p(out), self._p(o1), self._p(floor), _code(out), self._p(weight), _code(weight),
                   self._p(gate_pre), ctypes.c_long(gate_pre.stride(0)), ctypes.c_float(eps), ctypes.c_float(tiny), t, heads, vdim)

    # ---- a norm on a sublayer's output and the average over the layers' results (csrc/elementwise.cu)
    def out_norm_add(self, dst, src, y, bias, weight, eps, offset, hist=None, n_hist=0, coef=None, avg=None, cast=None) -> None:
        """dst = src + N(y + bias) (y None: dst = src); with `hist` float32 [>= n_hist, rows, dim], whose entry n_hist - 1 is
        dst: avg = sum_j coef[j] hist[j]; `cast` gets what goes on (avg, else dst) in its own dtype."""
        self._check(dst, src, y, bias, weight, hist, coef, avg, cast)
        self._f32("out_norm_add", dst, src, hist, coef, avg)
        rows, dim = dst.shape
        if src.shape != dst.shape or (y is not None and (y.shape != dst.shape or weight is None or weight.shape != (dim,))) \
                or (bias is not None and bias.shape != (dim,)) or (cast is not None and cast.shape != dst.shape) \
                or (hist is not None and (hist.shape[1:] != dst.shape or not 1 <= n_hist <= hist.shape[0] or coef is None
                                          or coef.shape[0] < n_hist or avg is None or avg.shape != dst.shape)):
            raise KernelError("out_norm_add: dst, src, y, avg, cast [rows, dim], bias and weight [dim], hist [n, rows, dim], coef [n]")
        self._call("hb_out_norm_add", self._p(dst), self._p(src), self._p(y), _code(y) if y is not None else 0, self._p(bias),
                   _code(bias) if bias is not None else 0, self._p(weight), _code(weight) if weight is not None else 0,
                   ctypes.c_float(eps), ctypes.c_float(offset), self._p(hist), ctypes.c_long(rows * dim), int(n_hist),
                   self._p(coef), self._p(avg), self._p(cast), _code(cast) if cast is not None else 0, rows, dim)

    # ---- attention whose heads share their weights after the softmax (csrc/attention_talking.cu)
    def qkv_talking_prepare(self, q_out, kv, keep, qkv, bias, q_weight, k_weight, eps, positions, table, rot_dims, interleaved,
                            first, blend, write_index, heads, kv_heads, key_dim, value_dim) -> None:
        self._check(q_out, kv, keep, qkv, bias, q_weight, k_weight, positions, table, first, blend, write_index)
        self._f32("qkv_talking_prepare", keep, table, first, blend)
        t = qkv.shape[0]
        width = heads * key_dim + kv_heads * (key_dim + value_dim)
        if qkv.shape != (t, width) or q_out.shape != (t, heads, key_dim) or q_out.dtype != qkv.dtype \
                or (kv is not None and (kv.dtype != qkv.dtype or kv.shape[1] != kv_heads or kv.shape[3] != key_dim + value_dim
                                        or write_index is None)) \
                or (bias is not None and bias.shape != (width,)) \
                or (q_weight is not None and (q_weight.shape != (key_dim,) or k_weight is None or k_weight.dtype != q_weight.dtype)) \
                or (keep is not None and keep.shape != (t, kv_heads, value_dim)) \
                or (first is not None and first.shape != (t, kv_heads, value_dim)) \
                or (rot_dims and (table is None or table.shape[1] != rot_dims)):
            raise KernelError("qkv_talking_prepare: qkv [tokens, q | k | v], q_out [tokens, heads, key_dim], cache [pages, "
                              "kv_heads, page, key_dim + value_dim], keep and first float32 [tokens, kv_heads, value_dim]")
        self._call("hb_qkv_talking_prepare", self._p(q_out), self._p(kv), self._p(keep), self._p(qkv), _code(qkv), self._p(bias),
                   _code(bias) if bias is not None else 0, self._p(q_weight), self._p(k_weight),
                   _code(q_weight) if q_weight is not None else 0, ctypes.c_float(eps), self._i32(positions, "positions"),
                   self._p(table), int(rot_dims), table.shape[0] if table is not None else 0, int(bool(interleaved)),
                   self._p(first), self._p(blend), self._i32(write_index, "write_index"),
                   kv.shape[0] - 1 if kv is not None else 0, kv.shape[2] if kv is not None else 1, t, heads, kv_heads,
                   key_dim, value_dim)

    TALKING_SPLIT_KEYS = 64                   # the fewest keys a part of a one-token row's keys holds

    def attention_talking(self, out, q, kv, block_table, rows, scale, head_scale, chunk, window, talk) -> None:
        """bfloat16 with keys and values of 128 numbers and pages of a multiple of 64 tokens: rows of several tokens run on the tcgen05 prompt kernel, every query head over the values of every kv
        head, and a second kernel mixes the heads; rows of one token, other sizes and float32 run on CUDA cores, rows
        of one token with their keys in parts where that fills more of the GPU."""
        self._check(out, q, kv, block_table, rows.row_slot, rows.query_start, rows.kv_len, head_scale, talk)
        self._f32("attention_talking", head_scale, talk)
        t, heads, kd = q.shape
        vd = out.shape[2]
        kv_heads = kv.shape[1]
        if out.shape != (t, heads, vd) or kv.shape[3] != kd + vd or not (out.dtype == q.dtype == kv.dtype) \
                or (head_scale is not None and head_scale.shape != (heads,)) or (talk is not None and talk.shape != (heads, heads)):
            raise KernelError("attention_talking: q [tokens, heads, key_dim], out [tokens, heads, value_dim], cache [pages, "
                              "kv_heads, page, key_dim + value_dim], head_scale [heads], talk [heads, heads]")
        common = (self._i32(block_table, "block_table"), block_table.shape[1], self._i32(rows.row_slot, "row_slot"),
                  self._i32(rows.query_start, "query_start"), self._i32(rows.kv_len, "kv_len"))
        n_rows, n_tokens = rows.n_rows, t
        fast = q.dtype == torch.bfloat16 and kd == 128 and vd == 128 and kv.shape[2] % 64 == 0 and scale > 0 \
            and self.attention_bf16 == "fast" \
            and self.prefill_attention == "tcgen05" and rows.n_rows > rows.n_decode
        if fast:
            value_heads = kv_heads if talk is not None else 1
            wide = out if value_heads == 1 and talk is None else torch.empty(t, heads * value_heads, vd, dtype=q.dtype, device=q.device)
            tile_q, tiles = 256, self._query_tiles(rows, 256)
            if self.prefill_tile == 128 or (self.prefill_tile is None and 4 * heads * value_heads * tiles < 3 * self.sms):
                tile_q, tiles = 128, self._query_tiles(rows, 128)
            self._call("hb_attention_prefill_tcgen05_rows", self._p(wide), self._p(q), self._p(kv), *common, rows.n_decode,
                       rows.n_rows, tiles, t, heads, kv_heads, kd, kv.shape[0] - 1, kv.shape[2], ctypes.c_float(scale), int(window),
                       tile_q, self._p(None), 1, value_heads, int(chunk), self._p(head_scale))
            if wide is not out:
                self._call("hb_talking_mix", self._p(out), self._p(wide), _code(q), rows.n_decode, t - rows.n_decode, heads,
                           kv_heads, vd, self._p(talk))
            n_rows = n_tokens = rows.n_decode                         # (rows of one token come first in a step)
            if not n_rows:
                return
        splits, partial = 1, None
        if n_rows == rows.n_decode and n_rows:                        # rows of one token only: their keys in parts
            keys = min(x for x in (rows.max_kv, chunk, window) if x > 0)
            splits = max(1, min(-(-self.sms // n_tokens), -(-keys // self.TALKING_SPLIT_KEYS), 64))   # about a block an SM
            if splits > 1:
                partial = torch.empty(n_tokens * splits * heads * (kv_heads * vd + 2), dtype=torch.float32, device=q.device)
        self._call("hb_attention_talking", self._p(out), self._p(q), self._p(kv), _code(q), *common, n_rows, n_tokens, heads,
                   kv_heads, kd, vd, kv.shape[0] - 1, kv.shape[2], ctypes.c_float(scale), self._p(head_scale), int(chunk),
                   int(window), self._p(talk), self._p(partial), splits)

    def feed_tokens(self, token_ids, last_tokens, rows, from_last) -> None:
        """token_ids[first token of row r] = last_tokens[slot of row r] for the rows whose `from_last` is set."""
        self._check(token_ids, last_tokens, rows.row_slot, rows.query_start, from_last)
        self._call("hb_feed_tokens", self._i32(token_ids, "token_ids"), self._i32(last_tokens, "last_tokens"),
                   self._i32(rows.row_slot, "row_slot"), self._i32(rows.query_start, "query_start"),
                   self._i32(from_last, "from_last"), rows.n_rows)

    def scatter_rows(self, table, slots, rows) -> None:
        """table[slots[i], :] = rows[i, :]: block-table rows that changed on the host, packed in the step's upload."""
        self._check(table, slots, rows)
        n, width = slots.shape[0], table.shape[1]
        if rows.shape[0] != n * width:
            raise KernelError(f"scatter_rows: {n} rows of {width} need {n * width} values, not {rows.shape[0]}")
        self._call("hb_scatter_rows", self._i32(table, "table"), self._i32(slots, "slots"), self._i32(rows, "rows"),
                   n, width, table.shape[0])

    def store_tokens(self, last_tokens, slots, tokens, n) -> None:
        """last_tokens[slots[i]] = tokens[i] for i < n."""
        self._check(last_tokens, slots, tokens)
        self._call("hb_store_tokens", self._i32(last_tokens, "last_tokens"), self._i32(slots, "slots"),
                   self._i32(tokens, "tokens"), int(n))

    def logprobs(self, chosen, top_ids, top, logits, tokens) -> None:
        """chosen [rows] float32: log softmax(logits)[tokens]; top_ids int32 / top float32 [rows, k]: the k most likely."""
        self._check(chosen, top_ids, top, logits, tokens)
        r, v = logits.shape
        k = top.shape[1]
        if logits.dtype != torch.float32 or chosen.dtype != torch.float32 or top.dtype != torch.float32 \
                or top_ids.dtype != torch.int32 or tokens.dtype != torch.int32:
            raise KernelError("logprobs: logits, chosen, top float32; top_ids, tokens int32")
        if chosen.shape[0] < r or tokens.shape[0] < r or top.shape != (r, k) or top_ids.shape != (r, k):
            raise KernelError("logprobs: chosen and tokens [rows], top_ids and top [rows, k]")
        self._call("hb_logprobs", self._p(chosen), self._p(top_ids), self._p(top), self._p(logits), self._p(tokens), r, v, k)

    def sample(self, tokens, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, position, filtered) -> None:
        self._check(tokens, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, position)
        r, v = logits.shape
        if logits.dtype != torch.float32 or tokens.dtype != torch.int32 or tokens.shape[0] < r:
            raise KernelError("sample: logits float32 [rows, vocab], tokens int32 [rows]")
        for name, t, dt in (("temperature", temperature, torch.float32), ("top_p", top_p, torch.float32),
                            ("min_p", min_p, torch.float32), ("top_k", top_k, torch.int32),
                            ("seed_lo", seed_lo, torch.int32), ("seed_hi", seed_hi, torch.int32),
                            ("position", position, torch.int32)):
            if t.dtype != dt or t.shape[0] < r:
                raise KernelError(f"sample: {name} must be {dt} [rows]")
        self._call("hb_sample", self._p(tokens), self._p(logits), self._p(temperature), self._p(top_k),
                   self._p(top_p), self._p(min_p), self._p(seed_lo), self._p(seed_hi), self._p(position),
                   int(bool(filtered)), r, v)
