"""Python face of the hand-written CUDA kernels.

Each method checks what the kernel cannot check for itself (device, dtype, contiguity), passes raw
pointers and the current stream to an `extern "C"` launcher, and raises `KernelError` with the
kernel's own message when it refuses a size. There is no other implementation behind these
methods: without a CUDA device or without the compiled library they raise, they never fall back
to library or CPU code.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dt}") from None


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


class RowScale:
    """A per-token scalar that a consumer of partial sums still has to multiply in: the 1/rms of a
    norm whose weight is already in the product's operand. sumsq: float32 [tokens, parts], the parts
    of every token's sum of squares; the scalar is 1 / sqrt(sum(parts) / dim + eps)."""

    def __init__(self, sumsq: torch.Tensor, dim: int, eps: float):
        assert sumsq.dtype == torch.float32 and sumsq.dim() == 2 and sumsq.is_contiguous()
        self.sumsq, self.dim, self.eps = sumsq, int(dim), float(eps)

    def args(self):
        return (_ptr(self.sumsq), c_int(self.sumsq.shape[1]), c_float(1.0 / self.dim), c_float(self.eps))


_NO_ROW_SCALE = (c_void_p(0), c_int(0), c_float(0.0), c_float(0.0))


def _row_scale_args(rs: Optional["RowScale"]):
    return _NO_ROW_SCALE if rs is None else rs.args()


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, rows_contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor (the kernels have no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if rows_contiguous and t.dim() >= 1 and t.stride(-1) != 1 and t.shape[-1] != 1:
        raise KernelError(f"{name}: last dimension must be contiguous")


class CudaOps:
    """Loads a kernel library on first use of an op that lives in it."""

    def __init__(self):
        self._libs = {}
        self.launches = 0  # kernels launched through this object (a counter for measurements)
        self.tensor_cores = True  # bfloat16 products on tcgen05 where the operands allow it
        self.tcgen05_attention = True  # prompt portions: attention on tcgen05 where the geometry allows it
        self.tma_decode_attention = True  # single decoded tokens: keys and values by TMA where the geometry allows it
        self.fused_decode_attention = True  # ... with the sum of the q|k|v parts, rotation and cache write in the same kernel
        self.latent_tensor_cores = True  # latent attention on mma.sync where the geometry allows it (off: CUDA cores)
        self.gated_attention_tensor_cores = True  # gated attention on mma.sync where the geometry allows it (off: CUDA cores)
        self.routed_tensor_cores = True  # per-expert products of a routed feed-forward on mma.sync (off: CUDA cores)
        # Steps of few tokens: products that add their K pieces themselves, with the norm before, the residual sum
        # and SiLU * up folded in (gemm_few_tokens). Off: measured on B200 (batch 8, 2,048-token contexts, 1B layer
        # sizes) such a step takes 1.15 ms with the pieces meeting inside clusters and 1.40 ms with them meeting in
        # global memory, against 0.89 ms with partial sums in memory that the norm and activation kernels add.
        self.few_token_products = False
        # Prompt-sized steps: the last product of a sub-layer adds itself into the residual stream in its
        # epilogue (gemm_add_into) instead of writing float32 results that the next norm reads back.
        # Bit-equal and off: the norms of a 2,048-token step get 150 us shorter (they read the stream
        # alone), but the products that read the stream in their epilogue, a thread a row, get 390 us
        # longer (5.43 against 5.03 ms a step at the Llama 3.2 1B sizes).
        self.add_into_stream = False
        # Steps of few tokens: the last product of a sub-layer adds its K splits inside itself (the CTA of
        # each tile of outputs that finishes last), adds the sum into the residual stream and leaves
        # weight * stream and the rows' sums of squares for the norm that follows, which then is no kernel
        # of its own: its 1/rms is multiplied in where the next product's partial sums are consumed.
        # Correct (tests/test_meet_products_gpu.py, and the engine's tests with it switched on) and off:
        # a decode step of batch 8 at the Llama 3.2 1B sizes takes 1.22 ms with it against 0.87 ms
        # without. The finishing CTA's tail (fence, counter, reading the other splits back from L2) is
        # as long as the norm kernel it replaces, and while the norm kernel ran, the CTAs of the next
        # product were already resident and fetching weights, which they cannot be beside this product's
        # CTAs (shared memory). It also moves the bfloat16 rounding of a norm's output (weight * x is
        # rounded before 1/rms is applied), so steps of few tokens and prompt steps would no longer
        # round alike.
        self.meet_products = False
        self._few_cache = {}
        self._err_host: Optional[torch.Tensor] = None  # pinned word that queue_error_check copies the kernels' error code into

    # ------------------------------------------------------------------ loading
    def lib(self, name: str = "core"):
        lib = self._libs.get(name)
        if lib is None:
            if not torch.cuda.is_available():
                raise KernelError("no CUDA device: this engine runs only on its CUDA kernels")
            path = _build.kernel_library_path(name)
            lib = ctypes.CDLL(path)
            lib.llm_last_error.restype = ctypes.c_char_p
            if name == "tensorcore":
                lib.llm_attention_mma_scratch_floats.restype = ctypes.c_longlong
                lib.llm_latent_attention_scratch_floats.restype = ctypes.c_longlong
                lib.llm_gemm_decode_scratch_floats.restype = ctypes.c_longlong
                # "auto", "on" or "off" (see use_cta_pairs; for measurements, pairs are not safe to serve with)
                pairs = os.environ.get("LLMENGINE_CTA_PAIRS", "").strip().lower()
                if pairs in ("auto", "on", "off"):
                    lib.llm_gemm_tc_pair(c_int({"auto": -1, "on": 1, "off": 0}[pairs]))
            self._libs[name] = lib
        return lib

    def use_cta_pairs(self, on) -> None:
        """Products of more than 128 tokens on CTA pairs (tcgen05 cta_group::2: two SMs share one
        256 x 256 tile and each loads half of the weight tile): True always, False or None never
        (the default), "auto" where the kernel library estimates them to be faster (long products
        and those of many rounds of tiles, e.g. gate|up and down of a 2,048-token prompt, not
        q|k|v or o). They are off by default because a prompt step at the Llama 3.2 3B layer sizes
        was seen to stop inside the pair kernel, rarely and for a cause that was not found."""
        mode = -1 if on == "auto" else (1 if on else 0)
        self.lib("tensorcore").llm_gemm_tc_pair(c_int(mode))

    GEMM_FORMS = ("one tile a CTA", "persistent, tiles of 256", "persistent, tiles of 192", "CTA pairs")

    def gemm_form(self, m: int, n: int, k: int, swiglu: bool = False) -> str:
        """Which tcgen05 kernel a product of more than SWAP_MAX_TOKENS tokens with n outputs (gate and
        up rows together when `swiglu`) runs on: one of GEMM_FORMS."""
        return self.GEMM_FORMS[int(self.lib("tensorcore").llm_gemm_tc_form(c_int(m), c_int(n), c_int(k), c_int(1 if swiglu else 0)))]

    def merge_splits_in_cluster(self, on: bool) -> None:
        """Decoding attention split over the keys: the CTAs of one (request, kv head) form a thread-block
        cluster and send their partial results to its first CTA through shared memory (on, the
        default), or write them to global memory where the last CTA to arrive adds them (off; more
        than eight splits always end that way, cluster by cluster)."""
        self.lib("tensorcore").llm_attention_decode_cluster_merge(c_int(1 if on else 0))

    def _check(self, rc: int, lib) -> None:
        self.launches += 1
        if rc != 0:
            raise KernelError(lib.llm_last_error().decode())

    # ------------------------------------------------------------------ elementwise
    def embed(self, table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, sumsq: Optional[torch.Tensor] = None,
              next_w: Optional[torch.Tensor] = None, scaled: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
        """out[n,:] (float32) = table[ids[n],:] * scale; sumsq[n] (float32, optional) = sum of the row's squares;
        scaled[n,:] (bfloat16, optional, with next_w float32 [dim]) = next_w * out[n,:]."""
        _need(table, "embed.table"); _need(ids, "embed.ids", torch.int32); _need(out, "embed.out", torch.float32)
        lib = self.lib()
        n, dim = out.shape
        assert table.shape[1] == dim and table.is_contiguous() and out.is_contiguous() and ids.numel() >= n
        if sumsq is not None:
            _need(sumsq, "embed.sumsq", torch.float32)
            assert sumsq.is_contiguous() and sumsq.numel() >= n
        ld_scaled = 0
        if scaled is not None:
            _need(scaled, "embed.scaled", torch.bfloat16); _need(next_w, "embed.next_w", torch.float32)
            assert scaled.shape[0] >= n and scaled.shape[1] == dim and next_w.numel() == dim and next_w.is_contiguous()
            ld_scaled = scaled.stride(0)
        self._check(lib.llm_embed(_ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), _ptr(out), _ptr(sumsq), c_int(n),
                                  c_int(dim), c_int(table.shape[0]), _ptr(next_w if scaled is not None else None), _ptr(scaled),
                                  c_longlong(ld_scaled), c_float(scale), _stream()), lib)
        return out

    def rmsnorm(self, h: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None, write_back: bool = True, center: bool = False) -> torch.Tensor:
        """x = h[r] (+ delta[r], or + sum_p delta[p][r] for a 3-d delta); out = (w*x)/rms(x), or with `center` (a layer norm
        without bias) out = w * (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps).
        With `delta` and write_back, h[r] is replaced by x (the fused residual sum).
        With `rows` (int32), output row i reads source row rows[i] and h is left as it is."""
        _need(h, "rmsnorm.h", torch.float32); _need(weight, "rmsnorm.weight", torch.float32); _need(out, "rmsnorm.out")
        lib = self.lib()
        dim = h.shape[-1]
        n_out = (rows.numel() if n_rows is None else n_rows) if rows is not None else (h.shape[0] if n_rows is None else n_rows)
        assert h.is_contiguous() and out.is_contiguous() and weight.numel() == dim and out.shape[-1] == dim
        assert out.shape[0] >= n_out
        n_part, pstride = 0, 0
        if delta is not None:
            _need(delta, "rmsnorm.delta", torch.float32)
            assert delta.is_contiguous() and delta.shape[-1] == dim
            n_part, pstride = (delta.shape[0], delta.stride(0)) if delta.dim() == 3 else (1, 0)
        if rows is not None:
            _need(rows, "rmsnorm.rows", torch.int32)
            write_back = False
        self._check(lib.llm_rmsnorm(_ptr(h), _ptr(delta), c_int(n_part), c_longlong(pstride), _ptr(weight),
                                    _ptr(rows), _ptr(out), c_int(dtype_code(out.dtype)), c_int(n_out), c_int(dim),
                                    c_float(eps), c_int(1 if (write_back and delta is not None) else 0),
                                    c_int(1 if center else 0), _stream()), lib)
        return out

    def residual_add(self, h: torch.Tensor, delta: torch.Tensor, n_rows: Optional[int] = None) -> torch.Tensor:
        _need(h, "residual_add.h", torch.float32); _need(delta, "residual_add.delta", torch.float32)
        lib = self.lib()
        assert h.is_contiguous() and delta.is_contiguous()
        n = (h.shape[0] if n_rows is None else n_rows) * h.shape[-1]
        n_part, pstride = (delta.shape[0], delta.stride(0)) if delta.dim() == 3 else (1, 0)
        self._check(lib.llm_residual_add(_ptr(h), _ptr(delta), c_int(n_part), c_longlong(pstride), c_longlong(n),
                                         _stream()), lib)
        return h

    def softcap(self, x: torch.Tensor, cap: float) -> torch.Tensor:
        """x <- cap * tanh(x / cap) in place (float32)."""
        _need(x, "softcap.x", torch.float32)
        assert x.is_contiguous() and cap > 0
        lib = self.lib()
        self._check(lib.llm_softcap(_ptr(x), c_longlong(x.numel()), c_float(cap), _stream()), lib)
        return x

    # what a gated feed-forward may apply to its gate; "clamped_swish" comes as ("clamped_swish", limit, slope):
    # g <- min(g, limit), u <- clamp(u, -limit, limit), g * sigmoid(slope * g) * (u + 1)
    ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}

    @classmethod
    def _act_args(cls, act):
        if isinstance(act, tuple):
            return c_int(cls.ACTIVATIONS[act[0]]), c_float(act[1]), c_float(act[2])
        return c_int(cls.ACTIVATIONS[act]), c_float(0.0), c_float(1.0)

    def silu_mul(self, gate_up: torch.Tensor, out: torch.Tensor, block: int = 0, act: str = "silu") -> torch.Tensor:
        """gate_up [n, 2*ff] -> out [n, ff] = act(gate)*up. block 0: gate columns first, then up;
        block b: blocks of 2b columns, b of gate followed by the b matching ones of up."""
        _need(gate_up, "silu_mul.in"); _need(out, "silu_mul.out", gate_up.dtype)
        lib = self.lib()
        n, ff = out.shape
        assert gate_up.is_contiguous() and out.is_contiguous() and gate_up.shape == (n, 2 * ff)
        self._check(lib.llm_silu_mul(_ptr(gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(n), c_int(ff),
                                     c_int(block), *self._act_args(act), _stream()), lib)
        return out

    EPILOGUE_ACTIVATIONS = ("silu", "gelu_tanh", "clamped_swish")  # what the gate|up product applies in its own epilogue (gemm_swiglu)

    def gemm_swiglu(self, a: torch.Tensor, w_blocked: torch.Tensor, out: torch.Tensor, ws=None,
                    row_scale: Optional[RowScale] = None, act: str = "silu") -> torch.Tensor:
        """out [m, ff] = silu(gate) * up where gate | up = a @ w_blocked.T and w_blocked [2*ff, k] holds
        blocks of 128 gate rows followed by the 128 matching up rows. With many tokens in bfloat16
        the activation is applied in the product's epilogue and the [m, 2*ff] intermediate never
        exists; otherwise the product runs first (as partial sums when few tokens are in the step)."""
        _need(a, "gemm_swiglu.a"); _need(w_blocked, "gemm_swiglu.w", a.dtype); _need(out, "gemm_swiglu.out", a.dtype)
        m, k = a.shape
        ff = out.shape[1]
        assert w_blocked.shape == (2 * ff, k) and out.shape[0] == m and out.is_contiguous() and ff % 128 == 0
        if m > self.SWAP_MAX_TOKENS and (act[0] if isinstance(act, tuple) else act) in self.EPILOGUE_ACTIVATIONS and self._tc_usable(a, w_blocked):
            assert row_scale is None, "a row scale is applied where partial sums are consumed (few tokens)"
            lib = self.lib("tensorcore")
            self._check(lib.llm_gemm_tc_swiglu(_ptr(a), _ptr(w_blocked), _ptr(out), c_int(m), c_int(ff), c_int(k),
                                               c_longlong(a.stride(0)), c_longlong(w_blocked.stride(0)),
                                               c_longlong(out.stride(0)), *self._act_args(act), _stream()), lib)
            return out
        assert ws is not None, "gemm_swiglu needs a workspace when it cannot fuse"
        if m <= self.SWAP_MAX_TOKENS:
            return self.silu_mul_partials(self.gemm_partials(a, w_blocked, ws, "swiglu.parts"), out, block=128, row_scale=row_scale, act=act)
        assert row_scale is None, "a row scale is applied where partial sums are consumed (few tokens)"
        gate_up = ws.get("swiglu.gate_up", (m, 2 * ff), a.dtype)
        self.gemm(a, w_blocked, gate_up)
        return self.silu_mul(gate_up, out, block=128, act=act)

    # ------------------------------------------------------------------ matrix products
    # A weight-streaming product (few tokens) is bound by memory; measured on B200 it streams fastest
    # with several CTAs per SM, each with a short ring of stages; but every split adds a partial
    # result that the consumer has to read. The K range is cut until there are about this many CTAs
    # (each keeping at least two k-tiles of 64); with more than 32 tokens the partial results weigh
    # eight times as much and half as many CTAs do better (batch 64: 37.4 k against 36.5 k tokens/s).
    SPLIT_TARGET_CTAS = 296

    def _tc_usable(self, a: torch.Tensor, w: torch.Tensor) -> bool:
        """bfloat16 operands that the tensor-core kernel takes (16-byte aligned rows of K % 8 == 0)."""
        if a.dtype != torch.bfloat16 or not self.tensor_cores:
            return False
        lib = self.lib("tensorcore")
        return bool(lib.llm_gemm_tc_supported(_ptr(a), _ptr(w), c_int(a.shape[0]), c_int(w.shape[0]), c_int(a.shape[1]),
                                              c_longlong(a.stride(0)), c_longlong(w.stride(0))))

    def _splits_for(self, M: int, N: int, K: int) -> int:
        tiles, k_tiles = (N + 127) // 128, (K + 63) // 64
        if M > self.SWAP_MAX_TOKENS:
            return 1
        target = self.SPLIT_TARGET_CTAS if M <= 32 else self.SPLIT_TARGET_CTAS // 2
        want = min(max(1, -(-target // tiles)), max(1, k_tiles // 2))
        return int(self.lib("tensorcore").llm_gemm_tc_splits(c_int(K), c_int(want)))

    SWAP_MAX_TOKENS = 64  # up to here weights fill the accumulator lanes and tokens the columns

    def _gemm_tc(self, a, w, out, splits: int = 1, split_stride: int = 0) -> None:
        M, K = a.shape
        N = w.shape[0]
        swap = 1 if M <= self.SWAP_MAX_TOKENS else 0
        lib = self.lib("tensorcore")
        ldo = out.stride(-2)
        self._check(lib.llm_gemm_tc(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)),
                                    c_longlong(w.stride(0)), c_longlong(ldo), c_int(dtype_code(out.dtype)), c_int(swap),
                                    c_int(splits), c_longlong(split_stride), c_int(3 if swap else 8), _stream()), lib)

    def gemm(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, ws=None) -> torch.Tensor:
        """out[m,n] = sum_k a[m,k]*w[n,k]; float32 accumulation; a and w of one dtype; out float32
        or that dtype. Rows may be strided views. bfloat16 runs on the tensor cores (with a
        workspace `ws`: cut along K and reduced when few tokens stream a weight with few output
        tiles); float32 on CUDA cores, every output element summed over k in ascending order
        whatever the batch."""
        _need(a, "gemm.a"); _need(w, "gemm.w", a.dtype); _need(out, "gemm.out")
        M, K = a.shape
        N = w.shape[0]
        assert w.shape[1] == K and out.shape == (M, N)
        if self._tc_usable(a, w):
            splits = self._splits_for(M, N, K) if (ws is not None and out.is_contiguous()) else 1
            if splits == 1:
                self._gemm_tc(a, w, out)
            else:
                parts = ws.get("gemm.parts", (splits, M, N), torch.float32)
                self._gemm_tc(a, w, parts, splits, M * N)
                self.reduce_partials(parts, out)
            return out
        lib = self.lib()
        self._check(lib.llm_gemm_simt(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K),
                                      c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)),
                                      c_int(dtype_code(a.dtype)), c_int(dtype_code(out.dtype)), _stream()), lib)
        return out

    def gemm_heads(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None,
                   gate_off: int = 0) -> bool:
        """out[:, h, :] = a[:, h, :] @ w[h].T for all heads in one tensor-core launch (a [n, H, K], w [H, N, K], out
        [n, H, N] bfloat16; views whose last dimension is contiguous); with gate (float32 partial sums [p, n, width]),
        times sigmoid(sum_p gate[p, t, gate_off + h*N + j]). False, with nothing done, when the operands are not what
        that kernel takes (the caller then uses heads_product)."""
        if a.dtype != torch.bfloat16 or not self.tensor_cores or a.stride(2) != 1 or out.stride(2) != 1:
            return False
        n, H, K = a.shape
        N = w.shape[1]
        assert w.shape == (H, N, K) and w.is_contiguous() and out.shape == (n, H, N) and w.dtype == a.dtype == out.dtype
        lib = self.lib("tensorcore")
        if not lib.llm_heads_product_mma_supported(_ptr(a), c_longlong(a.stride(0)), c_longlong(a.stride(1)), _ptr(w), c_int(K)):
            return False
        gargs = (c_void_p(0), c_int(0), c_longlong(0), c_int(0), c_int(0))
        if gate is not None:
            _need(gate, "gemm_heads.gate", torch.float32)
            assert gate.is_contiguous() and gate.dim() == 3 and gate.shape[1] >= n and gate_off + H * N <= gate.shape[2]
            gargs = (_ptr(gate), c_int(gate.shape[0]), c_longlong(gate.stride(0)), c_int(gate.shape[2]), c_int(gate_off))
        self._check(lib.llm_heads_product_mma(_ptr(a), c_longlong(a.stride(0)), c_longlong(a.stride(1)), _ptr(w), _ptr(out),
                                              c_longlong(out.stride(0)), c_longlong(out.stride(1)), c_int(n), c_int(H), c_int(N), c_int(K),
                                              *gargs, _stream()), lib)
        return True

    def gemm_partials(self, a: torch.Tensor, w: torch.Tensor, ws, tag: str) -> torch.Tensor:
        """As gemm, for consumers that add partial sums themselves: returns float32 [parts, M, N]
        (scratch `tag` of workspace `ws`); the product is the sum over parts, to be taken in index
        order. parts is 1 unless few tokens stream a weight with few output tiles."""
        _need(a, "gemm.a"); _need(w, "gemm.w", a.dtype)
        M, K = a.shape
        N = w.shape[0]
        assert w.shape[1] == K
        if self._tc_usable(a, w):
            splits = self._splits_for(M, N, K)
            parts = ws.get(tag, (splits, M, N), torch.float32)
            self._gemm_tc(a, w, parts, splits, M * N)
            return parts
        parts = ws.get(tag, (1, M, N), torch.float32)
        self.gemm(a, w, parts[0])
        return parts

    def can_add_into(self, a: torch.Tensor, w: torch.Tensor) -> bool:
        """Whether gemm_add_into takes these operands: more tokens than the swapped form holds, on the
        tensor-core kernel."""
        return self.add_into_stream and a.shape[0] > self.SWAP_MAX_TOKENS and self._tc_usable(a, w)

    def gemm_add_into(self, a: torch.Tensor, w: torch.Tensor, h: torch.Tensor) -> None:
        """h[:m] (float32) += a @ w.T for a prompt-sized step: the product's epilogue reads, adds to and
        writes the residual stream itself, so the product never goes to memory and the norm that
        follows reads the stream alone. The same float32 sums as adding the product afterwards."""
        _need(a, "gemm_add.a", torch.bfloat16); _need(w, "gemm_add.w", torch.bfloat16); _need(h, "gemm_add.h", torch.float32)
        M, K = a.shape
        N = w.shape[0]
        assert self.can_add_into(a, w) and w.shape[1] == K and h.shape[0] >= M and h.shape[1] == N
        lib = self.lib("tensorcore")
        self._check(lib.llm_gemm_tc_add(_ptr(a), _ptr(w), _ptr(h), c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)),
                                        c_longlong(w.stride(0)), c_longlong(h.stride(0)), c_int(8), _stream()), lib)

    def row_scale(self, sumsq: torch.Tensor, dim: int, eps: float) -> RowScale:
        return RowScale(sumsq, dim, eps)

    def can_meet(self, a: torch.Tensor, w: torch.Tensor) -> bool:
        """Whether gemm_meet / gemm_scaled take these operands (few tokens on the tensor-core kernel)."""
        return self.meet_products and a.shape[0] <= self.SWAP_MAX_TOKENS and self._tc_usable(a, w)

    def gemm_meet(self, a: torch.Tensor, w: torch.Tensor, h: torch.Tensor, ws, tag: str, next_w: Optional[torch.Tensor] = None,
                  scaled: Optional[torch.Tensor] = None, sumsq: Optional[torch.Tensor] = None) -> None:
        """h[:m] (float32 stream) += a @ w.T for m <= SWAP_MAX_TOKENS tokens, with the K splits of the product
        added inside it (in index order, by the CTA of each tile of outputs that finishes last), so that
        no other kernel has to read partial sums. Beside it, for the norm that follows: scaled[:m]
        (bfloat16) = next_w * h, the operand of the product behind that norm, and sumsq [m, ceil(n / 128)]
        (float32) = the parts of every row's sum of squares; the norm's 1/rms is owed by whoever consumes
        that product (RowScale)."""
        _need(a, "gemm_meet.a", torch.bfloat16); _need(w, "gemm_meet.w", torch.bfloat16); _need(h, "gemm_meet.h", torch.float32)
        M, K = a.shape
        N = w.shape[0]
        assert self.can_meet(a, w) and w.shape[1] == K and h.shape[0] >= M and h.shape[1] == N
        tiles = (N + 127) // 128
        splits = self._splits_for(M, N, K)
        parts = ws.get(tag, (splits, M, N), torch.float32)
        counters = ws.get_zeroed("gemm.meet_counters", (tiles,), torch.int32)
        n_sumsq = 0
        if sumsq is not None:
            _need(sumsq, "gemm_meet.sumsq", torch.float32)
            assert sumsq.is_contiguous() and sumsq.shape[0] >= M and sumsq.shape[1] == tiles
            n_sumsq = tiles
        if scaled is not None:
            _need(scaled, "gemm_meet.scaled", torch.bfloat16); _need(next_w, "gemm_meet.next_w", torch.float32)
            assert scaled.shape[0] >= M and scaled.shape[1] == N and next_w.numel() == N and next_w.is_contiguous()
        lib = self.lib("tensorcore")
        self._check(lib.llm_gemm_tc_meet(_ptr(a), _ptr(w), _ptr(parts), c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)),
                                         c_longlong(w.stride(0)), c_int(splits), _ptr(h), c_longlong(h.stride(0)),
                                         _ptr(next_w if scaled is not None else None), _ptr(scaled),
                                         c_longlong(scaled.stride(0) if scaled is not None else 0), _ptr(sumsq), c_int(n_sumsq),
                                         _ptr(counters), c_int(3), _stream()), lib)

    def gemm_scaled(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, row_scale: RowScale) -> torch.Tensor:
        """out [m, n] (float32) = (a @ w.T) * row_scale, for m <= SWAP_MAX_TOKENS tokens, in one kernel."""
        _need(a, "gemm_scaled.a", torch.bfloat16); _need(w, "gemm_scaled.w", torch.bfloat16); _need(out, "gemm_scaled.out", torch.float32)
        M, K = a.shape
        N = w.shape[0]
        assert self.can_meet(a, w) and w.shape[1] == K and out.shape == (M, N) and row_scale.sumsq.shape[0] >= M
        lib = self.lib("tensorcore")
        self._check(lib.llm_gemm_tc_scaled(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)),
                                           c_longlong(w.stride(0)), c_longlong(out.stride(0)), *row_scale.args(), c_int(3),
                                           _stream()), lib)
        return out

    # ------------------------------------------------------------------ products of a step with few tokens
    FEW_TOKENS = 64  # up to here the weights fill the accumulator lanes and the kernel below applies
    FEW_TOKENS_TARGET_CTAS = 296  # K pieces are chosen so that about this many CTAs stream the weights

    def few_token_splits(self, n: int, k: int, t: int, mode: str, in_cluster: bool = False) -> int:
        """K pieces that gemm_few_tokens will use: 0 if the kernel does not take these sizes. mode: "plain",
        "residual" or "swiglu" (n counts gate and up rows). in_cluster: the pieces are the CTAs of a
        thread-block cluster and meet in its shared memory (at most 8); else they meet in global memory."""
        if not self.tensor_cores or not self.few_token_products or not (1 <= t <= self.FEW_TOKENS) or k % 8:
            return 0
        key = (n, k, t, mode, in_cluster)
        hit = self._few_cache.get(key)
        if hit is None:
            hit = self._few_cache[key] = self._few_token_splits(n, k, t, mode, in_cluster)
        return hit

    def _few_token_splits(self, n: int, k: int, t: int, mode: str, in_cluster: bool) -> int:
        tiles = -(-n // (256 if mode == "swiglu" else 128))
        target = self.FEW_TOKENS_TARGET_CTAS if t <= 32 else self.FEW_TOKENS_TARGET_CTAS // 2
        want = max(1, min(8 if in_cluster else 32, -(-target // tiles), max(1, -(-k // 64) // 2)))
        if mode == "residual" and in_cluster:
            want = max(want, 2)
        return int(self.lib("tensorcore").llm_gemm_decode_splits(c_int(n), c_int(k), c_int(t), c_int(self._FEW_MODES[mode]), c_int(want),
                                                                 c_int(1 if in_cluster else 0)))

    _FEW_MODES = {"plain": 0, "residual": 1, "swiglu": 2}

    def gemm_few_tokens(self, w: torch.Tensor, out: torch.Tensor, mode: str = "plain", x: Optional[torch.Tensor] = None,
                        norm=None, sumsq_out: Optional[torch.Tensor] = None, n_tokens: Optional[int] = None, ws=None) -> torch.Tensor:
        """out <- x . w^T for at most FEW_TOKENS tokens, with the K pieces added inside the product (no
        partial sums for other kernels to add) and the work around the product folded in.
        Activations: `x` bf16 [t, k]; or `norm` = (h float32 [rows, k], sumsq float32 [rows, parts], weight
        float32 [k], eps, row list int32 [t] or None): the RMSNorm of those rows, which then is no
        kernel of its own.
        mode "plain": out [t, n] float32 or bf16. "residual": out is the float32 residual stream
        [t, n], the product is added to it in place, and sumsq_out [t, parts] receives the parts of
        the new rows' sums of squares (parts = sumsq_out.shape[1], as residual_sumsq_parts says).
        "swiglu": w holds blocks of 128 gate rows and the 128 matching up rows, out bf16 [t, n / 2].
        With a workspace `ws` the K pieces meet in global memory (scratch of the workspace; any number of
        pieces, no clusters); without, inside a thread-block cluster (up to 8 pieces)."""
        _need(w, "gemm_few.w", torch.bfloat16); _need(out, "gemm_few.out")
        n, k = w.shape
        lib = self.lib("tensorcore")
        if x is not None:
            _need(x, "gemm_few.x", torch.bfloat16)
            t = x.shape[0] if n_tokens is None else n_tokens
            assert x.shape[1] == k
            xb, xf, ldx, ss, nss, nw, eps, rows = _ptr(x), c_void_p(0), x.stride(0), c_void_p(0), 0, c_void_p(0), 0.0, c_void_p(0)
        else:
            h, sumsq, weight, eps, row_list = norm
            _need(h, "gemm_few.h", torch.float32); _need(sumsq, "gemm_few.sumsq", torch.float32); _need(weight, "gemm_few.norm_weight", torch.float32)
            assert h.shape[1] == k and weight.numel() == k and sumsq.dim() == 2 and sumsq.is_contiguous() and sumsq.shape[0] >= h.shape[0]
            t = (row_list.numel() if row_list is not None else h.shape[0]) if n_tokens is None else n_tokens
            if row_list is not None:
                _need(row_list, "gemm_few.rows", torch.int32)
            xb, xf, ldx, ss, nss, nw, rows = c_void_p(0), _ptr(h), h.stride(0), _ptr(sumsq), sumsq.shape[1], _ptr(weight), _ptr(row_list)
        assert out.shape[0] >= t and out.shape[1] == (n // 2 if mode == "swiglu" else n)
        in_cluster = ws is None
        splits = self.few_token_splits(n, k, t, mode, in_cluster)
        if splits == 0:
            raise KernelError(f"gemm_few_tokens: sizes not taken (tokens={t} n={n} k={k} mode={mode})")
        parts = counters = None
        if not in_cluster:  # (also with one piece: the residual form always writes its sums through the scratch)
            code = self._FEW_MODES[mode]
            floats = int(lib.llm_gemm_decode_scratch_floats(c_int(n), c_int(k), c_int(t), c_int(code), c_int(splits)))
            parts = ws.get("few_tokens.pieces", (max(floats, 4),), torch.float32)
            counters = ws.get_zeroed("few_tokens.counters", (max(int(lib.llm_gemm_decode_tiles(c_int(n), c_int(code))), 1024),), torch.int32)
        nso = 0
        if mode == "residual":
            _need(sumsq_out, "gemm_few.sumsq_out", torch.float32)
            assert sumsq_out.is_contiguous() and sumsq_out.shape[0] >= t
            nso = sumsq_out.shape[1]
        self._check(lib.llm_gemm_decode(_ptr(w), c_longlong(w.stride(0)), c_int(n), c_int(k), c_int(t), xb, xf, c_longlong(ldx), ss,
                                        c_int(nss), nw, c_float(eps), rows, c_int(self._FEW_MODES[mode]), _ptr(out),
                                        c_longlong(out.stride(0)), c_int(dtype_code(out.dtype)), _ptr(sumsq_out), c_int(nso),
                                        c_int(splits), _ptr(parts), c_longlong(0 if parts is None else parts.numel()), _ptr(counters), _stream()), lib)
        return out

    def residual_sumsq_parts(self, n: int, k: int, t: int, in_cluster: bool = False) -> int:
        """Parts of a row's sum of squares that gemm_few_tokens(mode="residual") writes for these sizes."""
        tiles = -(-n // 128)
        return tiles * self.few_token_splits(n, k, t, "residual", True) if in_cluster else tiles

    def reduce_partials(self, parts: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out = sum over parts[p] (index order); out float32 or bfloat16, contiguous."""
        _need(parts, "reduce.parts", torch.float32); _need(out, "reduce.out")
        assert parts.is_contiguous() and out.is_contiguous() and parts.dim() == 3 and parts.shape[1:] == out.shape
        lib = self.lib()
        self._check(lib.llm_reduce_partials(_ptr(parts), c_int(parts.shape[0]), c_longlong(parts.stride(0)), _ptr(out),
                                            c_int(dtype_code(out.dtype)), c_longlong(out.numel()), _stream()), lib)
        return out

    def silu_mul_partials(self, parts: torch.Tensor, out: torch.Tensor, block: int = 0,
                          row_scale: Optional[RowScale] = None, act: str = "silu") -> torch.Tensor:
        """parts float32 [p, n, 2*ff] (gate | up partial sums, columns laid out as in silu_mul)
        -> out [n, ff] = silu(gate) * up; with row_scale, gate and up of row n are first multiplied by it."""
        _need(parts, "silu_mul.parts", torch.float32); _need(out, "silu_mul.out")
        n, ff = out.shape
        assert parts.is_contiguous() and out.is_contiguous() and parts.shape[1:] == (n, 2 * ff)
        lib = self.lib()
        self._check(lib.llm_silu_mul_partials(_ptr(parts), c_int(parts.shape[0]), c_longlong(parts.stride(0)), _ptr(out),
                                              c_int(dtype_code(out.dtype)), c_int(n), c_int(ff), c_int(block),
                                              *_row_scale_args(row_scale), *self._act_args(act), _stream()), lib)
        return out

    def tensor_core_error(self) -> int:
        """Code left by a tensor-core kernel that gave up a bounded wait (0: none); reading clears it.
        Synchronizes."""
        if "tensorcore" not in self._libs:
            return 0
        return int(self._libs["tensorcore"].llm_gemm_tc_error())

    # What the codes mean (csrc/kernels/tc_common.cuh, attention_tc.cu, attention_decode.cu).
    ERROR_CODES = {1: "product: a stage never became free", 2: "product: operands or an accumulator never arrived",
                   3: "product: the accumulator was never finished", 4: "product: a copy in flight did not land",
                   11: "prompt attention: keys or values never arrived", 12: "prompt attention: scores or probabilities never arrived",
                   13: "prompt attention: the output product never finished",
                   21: "decoding attention: a stage never became free", 22: "decoding attention: a tile never arrived",
                   23: "decoding attention: a copy in flight did not land", 24: "decoding attention: a CTA of the cluster never reported"}

    def queue_error_check(self) -> None:
        """Queues, behind the kernels launched so far on the current stream, a copy of the tensor-core
        kernels' error word into pinned host memory (4 bytes; may be captured in a CUDA graph).
        take_step_error() reads it once the stream has been synchronized."""
        if "tensorcore" not in self._libs:
            return
        if self._err_host is None:
            self._err_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        lib = self._libs["tensorcore"]
        rc = lib.llm_tc_error_copy_async(c_void_p(self._err_host.data_ptr()), _stream())
        if rc != 0:
            raise KernelError(lib.llm_last_error().decode())

    def take_step_error(self) -> int:
        """The code that the last queued check brought back (0: none), without touching the device
        unless there is one: then the device's word is cleared, so that later kernels wait normally."""
        if self._err_host is None:
            return 0
        code = int(self._err_host[0])
        if code:
            self._err_host[0] = 0
            self.tensor_core_error()
        return code

    def set_tensor_core_error(self, code: int) -> None:
        """Writes the error word from the host, for tests of the error handling (no kernel has to
        fail for the host to see a code)."""
        rc = int(self.lib("tensorcore").llm_tc_error_set(c_int(code)))
        if rc != 0:
            raise KernelError(f"cannot write the error word ({rc})")

    # ------------------------------------------------------------------ attention
    def rope_kv_write(self, qkv: torch.Tensor, positions: torch.Tensor, token_seq: torch.Tensor,
                      block_table: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                      kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor], n_tokens: int, nq: int,
                      nkv: int, hd: int, parts: Optional[torch.Tensor] = None, row_scale: Optional[RowScale] = None) -> None:
        """Rotates q and k of qkv [n, (nq+2nkv)*hd] in place by the tables cos/sin [max_pos, hd/2]
        and writes k, v of each token into its page: kcache/vcache [pages, nkv, page_size, hd].
        With `parts` (float32 [p, n, width] partial sums of the q|k|v product) the values are the
        sums over parts (times row_scale, if given); then only the q section of qkv is written (k and v
        go to the cache)."""
        assert row_scale is None or parts is not None
        _need(qkv, "rope.qkv"); _need(positions, "rope.positions", torch.int32)
        _need(token_seq, "rope.token_seq", torch.int32); _need(block_table, "rope.block_table", torch.int32)
        page_size = 1
        if kcache is not None:
            _need(kcache, "rope.kcache", qkv.dtype); _need(vcache, "rope.vcache", qkv.dtype)
            assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape == vcache.shape
            assert kcache.shape[1] == nkv and kcache.shape[3] == hd
            page_size = kcache.shape[2]
        if cos is not None:
            _need(cos, "rope.cos", torch.float32); _need(sin, "rope.sin", torch.float32)
            assert cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] == hd // 2
        assert qkv.shape[1] == (nq + 2 * nkv) * hd and block_table.is_contiguous()
        lib = self.lib()
        n_parts, pstride = 0, 0
        if parts is not None:
            _need(parts, "rope.parts", torch.float32)
            assert parts.is_contiguous() and parts.dim() == 3 and parts.shape[2] == qkv.shape[1] and parts.shape[1] >= n_tokens
            n_parts, pstride = parts.shape[0], parts.stride(0)
        self._check(lib.llm_rope_kv_write(_ptr(qkv), c_longlong(qkv.stride(0)), c_int(dtype_code(qkv.dtype)),
                                          _ptr(parts), c_int(n_parts), c_longlong(pstride), _ptr(positions), _ptr(token_seq), _ptr(block_table),
                                          c_int(block_table.shape[1]), _ptr(cos), _ptr(sin), _ptr(kcache),
                                          _ptr(vcache), c_int(n_tokens), c_int(nq), c_int(nkv), c_int(hd),
                                          c_int(page_size), *_row_scale_args(row_scale), _stream()), lib)

    # decoding: the key range is cut at absolute multiples of `split_keys` (a multiple of 64); see _split_policy
    ATTENTION_TARGET_CTAS = 592
    ATTENTION_MAX_SPLITS = 128  # what the kernels' merge takes
    ATTENTION_MIN_SPLIT_KEYS = 320
    TC_ATTENTION_MIN_TOKENS = 32  # longest portion of the step from which the tcgen05 attention kernel is used
    TC_ATTENTION_MAX_BLOCKS = 4096  # widest block table whose slice it keeps in shared memory (wider: the mma.sync kernel)

    def _split_policy(self, pairs: int, max_seq_len: int, hd: int = 64):
        """-> (number of key splits, keys per split) of a step of single tokens with `pairs` (request,
        key/value head) pairs. Measured on B200 (head size 64): the cache streams fastest with four
        CTAs on each of the 148 SMs (592) and no split; with fewer pairs the range is cut to fill
        those places, but into pieces of at least ATTENTION_MIN_SPLIT_KEYS keys, since every split
        ends in a partial output and a merge. Up to 8 splits merge inside a thread-block cluster
        (2,048-token contexts at batch 8: 11.0 us, against 13.3 us through global memory); more run
        as several clusters of 8 whose results meet in global memory (one request of 16,384 tokens:
        48 splits, 16.4 us against 27.2 us with every split's partial in global memory). Inside a
        decode step 320 and 384 keys measure the same (0.881 ms), 256 keys 0.898 ms."""
        # head size 128: stages are twice as large, two CTAs with the long ring an SM do best (296 places)
        places = self.ATTENTION_TARGET_CTAS if hd <= 64 else max(1, self.ATTENTION_TARGET_CTAS // 2)
        want = min(self.ATTENTION_MAX_SPLITS, places // max(pairs, 1), max_seq_len // self.ATTENTION_MIN_SPLIT_KEYS)
        if want > 8:
            want = want // 8 * 8  # whole clusters of eight splits: a ninth split would cost a cluster of its own
        if want <= 1:
            return 1, 256
        split_keys = -(-(-(-max_seq_len // want)) // 64) * 64
        return -(-max_seq_len // split_keys), split_keys

    def _decode_splits(self, lib, batch, nq: int, nkv: int, hd: int):
        """How a step of single tokens cuts its key ranges -> (n_splits, split_keys, scratch, counters)."""
        n_splits, split_keys = self._split_policy(batch.n_seqs * nkv, batch.max_seq_len, hd)
        scratch = counters = None
        if n_splits > 1:
            floats = int(lib.llm_attention_mma_scratch_floats(c_int(batch.n_tokens), c_int(nq), c_int(hd), c_int(n_splits)))
            scratch = batch.ws.get("attention.splits", (floats,), torch.float32)
            counters = batch.ws.get_zeroed("attention.split_counters", (batch.n_seqs * nkv,), torch.int32)
        return n_splits, split_keys, scratch, counters

    def decode_attention_fusable(self, batch, kcache: torch.Tensor, nq: int, nkv: int, hd: int, out: torch.Tensor) -> bool:
        """Whether paged_attention_decode_fused takes this step: single tokens only, bfloat16, and a
        geometry of the TMA decoding kernel."""
        if not (self.fused_decode_attention and self.tma_decode_attention and self.tensor_cores and kcache.dtype == torch.bfloat16):
            return False
        if not (batch.max_new_tokens == 1 and batch.n_tokens == batch.n_seqs):
            return False
        lib = self.lib("tensorcore")
        if not lib.llm_attention_decode_supported(c_int(nq), c_int(nkv), c_int(hd), c_int(kcache.shape[2]), c_longlong(8),
                                                  c_longlong(out.stride(0))):
            return False
        return self._split_policy(batch.n_seqs * nkv, batch.max_seq_len, hd)[0] <= 128

    def paged_attention_decode_fused(self, parts: torch.Tensor, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                                     kcache: torch.Tensor, vcache: torch.Tensor, batch, block_table: torch.Tensor,
                                     out: torch.Tensor, nq: int, nkv: int, hd: int, scale: float, window: int = 0,
                                     row_scale: Optional[RowScale] = None) -> torch.Tensor:
        """A step of single tokens, from the q|k|v product's partial sums (float32 [p, n, (nq+2nkv)*hd],
        added in index order, times row_scale if given): rotation of q and k by cos/sin [positions, hd/2] (none if both are
        None), the write of k and v into the token's page, and attention over the cache, in one kernel."""
        _need(parts, "attention.parts", torch.float32); _need(kcache, "attention.kcache", torch.bfloat16)
        _need(vcache, "attention.vcache", torch.bfloat16); _need(out, "attention.out", torch.bfloat16)
        _need(block_table, "attention.block_table", torch.int32)
        assert parts.is_contiguous() and parts.dim() == 3 and parts.shape[2] == (nq + 2 * nkv) * hd and parts.shape[1] >= batch.n_tokens
        assert kcache.is_contiguous() and vcache.is_contiguous() and block_table.is_contiguous() and kcache.shape == vcache.shape
        assert kcache.shape[1] == nkv and kcache.shape[3] == hd
        if cos is not None:
            _need(cos, "attention.cos", torch.float32); _need(sin, "attention.sin", torch.float32)
            assert cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] == hd // 2 and cos.shape == sin.shape
            assert cos.shape[0] >= batch.max_seq_len
        lib = self.lib("tensorcore")
        n_splits, split_keys, scratch, counters = self._decode_splits(lib, batch, nq, nkv, hd)
        self._check(lib.llm_paged_attention_decode_fused(
            _ptr(parts), c_int(parts.shape[0]), c_longlong(parts.stride(0)), _ptr(cos), _ptr(sin), _ptr(kcache), _ptr(vcache),
            c_longlong(kcache.shape[0]), _ptr(batch.seq_start), _ptr(batch.seq_qoff), _ptr(block_table),
            c_int(block_table.shape[1]), _ptr(out), c_longlong(out.stride(0)), c_int(batch.n_seqs), c_int(nq), c_int(nkv),
            c_int(hd), c_int(kcache.shape[2]), c_float(scale), c_int(window), c_int(n_splits), c_int(split_keys),
            _ptr(scratch), _ptr(counters), *_row_scale_args(row_scale), _stream()), lib)
        return out

    def paged_attention(self, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, batch,
                        block_table: torch.Tensor, out: torch.Tensor, nq: int, nkv: int, hd: int, scale: float,
                        window: int = 0) -> torch.Tensor:
        """Causal attention of every token of the step over cache positions lo..pos of its request.
        q: rows of [nq*hd] (may be a view of the qkv buffer); out [n, nq*hd]; `batch` is the step
        context (positions, token_seq, seq_start, seq_ntok, seq_qoff, the counts, scratch).
        bfloat16 with head sizes 16/32/64/128 runs on tensor cores (with the key range cut into
        splits when every request brings one token); anything else on CUDA cores in float32."""
        _need(q, "attention.q"); _need(kcache, "attention.kcache", q.dtype); _need(vcache, "attention.vcache", q.dtype)
        _need(out, "attention.out", q.dtype); _need(block_table, "attention.block_table", torch.int32)
        assert kcache.is_contiguous() and vcache.is_contiguous() and block_table.is_contiguous()
        assert kcache.shape[1] == nkv and kcache.shape[3] == hd
        n_tokens, page = batch.n_tokens, kcache.shape[2]
        if q.dtype == torch.bfloat16 and self.tensor_cores:
            lib = self.lib("tensorcore")
            if (self.tcgen05_attention and batch.max_new_tokens >= self.TC_ATTENTION_MIN_TOKENS and
                    block_table.shape[1] <= self.TC_ATTENTION_MAX_BLOCKS and
                    lib.llm_attention_tc_supported(c_int(nq), c_int(nkv), c_int(hd), c_int(page), c_longlong(q.stride(0)),
                                                   c_longlong(out.stride(0)))):
                # prompt portions: tcgen05 kernel (128 rows per CTA, scores and output in tensor memory)
                work = batch.ws.get_zeroed("attention.work_counters", (2,), torch.int32)  # left at zero by the kernel
                self._check(lib.llm_paged_attention_tc(
                    _ptr(q), c_longlong(q.stride(0)), _ptr(kcache), _ptr(vcache), c_longlong(kcache.shape[0]),
                    _ptr(batch.seq_start), _ptr(batch.seq_ntok), _ptr(batch.seq_qoff), _ptr(block_table),
                    c_int(block_table.shape[1]), _ptr(out), c_longlong(out.stride(0)), c_int(batch.n_seqs),
                    c_int(batch.max_new_tokens), c_int(nq), c_int(nkv), c_int(hd), c_int(page), c_float(scale), c_int(window),
                    c_int(q.shape[0]), _ptr(work), _stream()), lib)
                return out
            decode_only = batch.max_new_tokens == 1 and batch.n_tokens == batch.n_seqs
            use_tma = decode_only and self.tma_decode_attention and lib.llm_attention_decode_supported(
                c_int(nq), c_int(nkv), c_int(hd), c_int(page), c_longlong(q.stride(0)), c_longlong(out.stride(0)))
            if use_tma or lib.llm_attention_mma_supported(c_int(nq), c_int(nkv), c_int(hd), c_longlong(q.stride(0)), c_longlong(out.stride(0))):
                n_splits, split_keys, scratch, counters = 1, 256, None, None
                if decode_only:
                    n_splits, split_keys, scratch, counters = self._decode_splits(lib, batch, nq, nkv, hd)
                if use_tma and n_splits <= 128:
                    # single decoded tokens: keys and values by TMA, one producer thread, four computing warps
                    self._check(lib.llm_paged_attention_decode(
                        _ptr(q), c_longlong(q.stride(0)), _ptr(kcache), _ptr(vcache), c_longlong(kcache.shape[0]),
                        _ptr(batch.seq_start), _ptr(batch.seq_qoff), _ptr(block_table), c_int(block_table.shape[1]), _ptr(out),
                        c_longlong(out.stride(0)), c_int(batch.n_seqs), c_int(nq), c_int(nkv), c_int(hd), c_int(page),
                        c_float(scale), c_int(window), c_int(n_splits), c_int(split_keys), _ptr(scratch), _ptr(counters),
                        _stream()), lib)
                    return out
                self._check(lib.llm_paged_attention_mma(
                    _ptr(q), c_longlong(q.stride(0)), _ptr(kcache), _ptr(vcache), _ptr(batch.seq_start), _ptr(batch.seq_ntok),
                    _ptr(batch.seq_qoff), _ptr(block_table), c_int(block_table.shape[1]), _ptr(out), c_longlong(out.stride(0)),
                    c_int(batch.n_seqs), c_int(n_tokens), c_int(batch.max_new_tokens), c_int(nq), c_int(nkv), c_int(hd),
                    c_int(page), c_float(scale), c_int(window), c_int(n_splits), c_int(split_keys),
                    _ptr(scratch), _stream()), lib)
                if n_splits > 1:
                    self.launches += 1  # the kernel that merges the splits
                return out
        lib = self.lib()
        self._check(lib.llm_paged_attention_simt(_ptr(q), c_longlong(q.stride(0)), _ptr(kcache), _ptr(vcache),
                                                 c_int(dtype_code(q.dtype)), _ptr(batch.positions), _ptr(batch.token_seq),
                                                 _ptr(block_table), c_int(block_table.shape[1]), _ptr(out),
                                                 c_longlong(out.stride(0)), c_int(n_tokens), c_int(nq), c_int(nkv),
                                                 c_int(hd), c_int(page), c_float(scale), c_int(window), _stream()), lib)
        return out

    def attention_kernels(self, nq: int, nkv: int, hd: int, page: int):
        """-> (what prompt portions of 32 tokens or more run on, what single decoded tokens run on) for
        a bfloat16 model of this geometry: "tensor cores" (tcgen05 for portions; TMA-fed mma.sync for
        decoding), "tensor cores (mma.sync, the general kernel)" or "CUDA cores"."""
        lib = self.lib("tensorcore")
        ld = nq * hd
        general = bool(lib.llm_attention_mma_supported(c_int(nq), c_int(nkv), c_int(hd), c_longlong(ld), c_longlong(ld)))
        fallback = "tensor cores (mma.sync, the general kernel)" if general else "CUDA cores"
        prompt = "tensor cores" if self.tcgen05_attention and lib.llm_attention_tc_supported(
            c_int(nq), c_int(nkv), c_int(hd), c_int(page), c_longlong(ld), c_longlong(ld)) else fallback
        decode = "tensor cores" if self.tma_decode_attention and lib.llm_attention_decode_supported(
            c_int(nq), c_int(nkv), c_int(hd), c_int(page), c_longlong(ld), c_longlong(ld)) else fallback
        if not self.tensor_cores:
            prompt = decode = "CUDA cores"
        return prompt, decode

    # ------------------------------------------------------------------ stream and token side input
    def stream_add(self, h: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor] = None,
                   copy: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> torch.Tensor:
        """h[:n] += a (+ b): float32 [n, dim] or [parts, n, dim] partial sums added in index order, a before b;
        copy[:n] (optional, float32 or bfloat16) = the new h, the stream as an operand of a product."""
        _need(h, "stream_add.h", torch.float32)
        n = h.shape[0] if n_rows is None else n_rows
        lib = self.lib()
        args = []
        for t, name in ((a, "a"), (b, "b")):
            if t is None:
                args += [c_void_p(0), c_int(0), c_longlong(0)]
                continue
            _need(t, "stream_add." + name, torch.float32)
            assert t.is_contiguous() and t.shape[-1] == h.shape[-1] and t.shape[-2] == h.shape[0]
            args += [_ptr(t), c_int(t.shape[0] if t.dim() == 3 else 1), c_longlong(t.stride(0) if t.dim() == 3 else 0)]
        code = F32
        if copy is not None:
            _need(copy, "stream_add.copy")
            assert copy.is_contiguous() and copy.shape[-1] == h.shape[-1] and copy.shape[0] >= n
            code = dtype_code(copy.dtype)
        assert h.is_contiguous()
        self._check(lib.llm_stream_add(_ptr(h), *args, _ptr(copy), c_int(code), c_longlong(n * h.shape[-1]), _stream()), lib)
        return h

    def token_gate(self, z: torch.Tensor, table: torch.Tensor, col0: int, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col0 + j]; z, out [n, dim] contiguous, of the table's dtype."""
        _need(z, "token_gate.z"); _need(table, "token_gate.table", z.dtype); _need(out, "token_gate.out", z.dtype)
        _need(ids, "token_gate.ids", torch.int32)
        n, dim = out.shape
        assert z.is_contiguous() and out.is_contiguous() and z.shape == out.shape and ids.numel() >= n
        lib = self.lib()
        self._check(lib.llm_token_gate(_ptr(z), _ptr(table), c_longlong(table.stride(0)), c_int(col0), _ptr(ids), c_int(table.shape[0]),
                                       _ptr(out), c_int(n), c_int(dim), c_int(dtype_code(z.dtype)), _stream()), lib)
        return out

    # ------------------------------------------------------------------ latent attention
    def latent_prep(self, parts: torch.Tensor, q_off: int, q_rank: int, kv_off: int, kv_rank: int, rot_dim: int, rot_dims: int,
                    wq: torch.Tensor, wkv: torch.Tensor, eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                    batch, block_table: torch.Tensor, cq: torch.Tensor, cache: Optional[torch.Tensor]) -> None:
        """From the float32 partial sums parts [p, n, width] of the mixer's first product: cq [n, q_rank] = the RMS-normed
        query latent (weight wq); the cache row [c | kr] of every token, c = the RMS-normed first kv_rank numbers of the
        key/value columns (weight wkv), kr = the next rot_dim with the first rot_dims rotated by cos/sin [positions, rot_dims/2].
        cache [pages, 1, page_size, kv_rank + rot_dim], or None for a run that writes none."""
        _need(parts, "latent_prep.parts", torch.float32); _need(cq, "latent_prep.cq"); _need(block_table, "latent_prep.block_table", torch.int32)
        _need(wq, "latent_prep.wq", torch.float32); _need(wkv, "latent_prep.wkv", torch.float32)
        n = batch.n_tokens
        assert parts.is_contiguous() and parts.dim() == 3 and parts.shape[1] >= n and block_table.is_contiguous()
        assert wq.numel() == q_rank and wkv.numel() == kv_rank and cq.shape[0] >= n and cq.shape[1] == q_rank
        page = 1
        if cache is not None:
            _need(cache, "latent_prep.cache", cq.dtype)
            assert cache.is_contiguous() and cache.shape[1] == 1 and cache.shape[3] == kv_rank + rot_dim
            page = cache.shape[2]
        if rot_dims:
            _need(cos, "latent_prep.cos", torch.float32); _need(sin, "latent_prep.sin", torch.float32)
            assert cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] == rot_dims // 2 and cos.shape == sin.shape
        lib = self.lib()
        self._check(lib.llm_latent_prep(_ptr(parts), c_int(parts.shape[0]), c_longlong(parts.stride(0)), c_int(parts.shape[2]),
                                        c_int(q_off), c_int(q_rank), c_int(kv_off), c_int(kv_rank), c_int(rot_dim), c_int(rot_dims),
                                        _ptr(wq), _ptr(wkv), c_float(eps), _ptr(cos), _ptr(sin), _ptr(batch.positions),
                                        _ptr(batch.token_seq), _ptr(block_table), c_int(block_table.shape[1]), _ptr(cq),
                                        c_longlong(cq.stride(0)), _ptr(cache), c_int(page), c_int(dtype_code(cq.dtype)), c_int(n),
                                        _stream()), lib)

    def heads_product(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor] = None,
                      gate_off: int = 0) -> torch.Tensor:
        """out[t, h, :] = w[h] a[t, h, :] for a [n, H, K], w [H, N, K], out [n, H, N] (views whose last dimension is
        contiguous); with gate (float32 partial sums [p, n, width]), times sigmoid(sum_p gate[p, t, gate_off + h*N + j])."""
        _need(a, "heads_product.a"); _need(w, "heads_product.w", a.dtype); _need(out, "heads_product.out", a.dtype)
        n, H, K = a.shape
        N = w.shape[1]
        assert w.shape == (H, N, K) and w.is_contiguous() and out.shape == (n, H, N)
        gargs = (c_void_p(0), c_int(0), c_longlong(0), c_int(0), c_int(0))
        if gate is not None:
            _need(gate, "heads_product.gate", torch.float32)
            assert gate.is_contiguous() and gate.dim() == 3 and gate.shape[1] >= n and gate_off + H * N <= gate.shape[2]
            gargs = (_ptr(gate), c_int(gate.shape[0]), c_longlong(gate.stride(0)), c_int(gate.shape[2]), c_int(gate_off))
        lib = self.lib()
        self._check(lib.llm_heads_product(_ptr(a), c_longlong(a.stride(0)), c_longlong(a.stride(1)), _ptr(w), c_longlong(K), _ptr(out),
                                          c_longlong(out.stride(0)), c_longlong(out.stride(1)), c_int(n), c_int(H), c_int(N), c_int(K),
                                          *gargs, c_int(dtype_code(a.dtype)), _stream()), lib)
        return out

    def latent_query(self, q: torch.Tensor, wkt: Optional[torch.Tensor], ql: torch.Tensor, heads: int, dim: int, rot_dim: int,
                     kv_rank: int, rot_dims: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                     absorb: bool = True) -> torch.Tensor:
        """q [n, H*(dim+rot_dim)] -> ql [n, H, kv_rank+rot_dim]: per head, wkt[h] (the head's key map transposed,
        [kv_rank, dim]) applied to the unrotated part, unless absorb is False (then the caller writes those columns),
        followed by the rotated part, its first rot_dims numbers turned by the token's position."""
        _need(q, "latent_query.q"); _need(ql, "latent_query.ql", q.dtype); _need(positions, "latent_query.positions", torch.int32)
        n = ql.shape[0]
        assert ql.is_contiguous() and ql.shape == (n, heads, kv_rank + rot_dim) and q.shape[1] == heads * (dim + rot_dim)
        if absorb:
            _need(wkt, "latent_query.wkt", q.dtype)
            assert wkt.is_contiguous() and wkt.shape == (heads, kv_rank, dim)
        lib = self.lib()
        self._check(lib.llm_latent_query(_ptr(q), c_longlong(q.stride(0)), _ptr(wkt), _ptr(ql), c_int(n), c_int(heads), c_int(dim),
                                         c_int(rot_dim), c_int(kv_rank), c_int(rot_dims), c_int(1 if absorb else 0), _ptr(cos), _ptr(sin),
                                         _ptr(positions), c_int(dtype_code(q.dtype)), _stream()), lib)
        return ql

    def latent_attention(self, ql: torch.Tensor, cache: torch.Tensor, batch, block_table: torch.Tensor, out: torch.Tensor,
                         kv_rank: int, scale: float, window: int = 0) -> torch.Tensor:
        """Causal softmax attention of every token of the step over the cached rows lo..pos of its request: ql [n, H, Dk]
        against cache [pages, 1, page_size, Dk]; the values are the first kv_rank numbers of the rows; out [n, H, kv_rank]."""
        _need(ql, "latent_attention.ql"); _need(cache, "latent_attention.cache", ql.dtype); _need(out, "latent_attention.out", ql.dtype)
        _need(block_table, "latent_attention.block_table", torch.int32)
        n, H, Dk = ql.shape
        assert ql.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and block_table.is_contiguous()
        assert cache.shape[1] == 1 and cache.shape[3] == Dk and out.shape == (n, H, kv_rank) and n >= batch.n_tokens
        if ql.dtype == torch.bfloat16 and self.tensor_cores and self.latent_tensor_cores:
            lib = self.lib("tensorcore")
            if lib.llm_latent_attention_mma_supported(c_int(H), c_int(kv_rank), c_int(Dk - kv_rank)):
                n_splits, split_keys, scratch = 1, 256, None
                if batch.max_new_tokens == 1 and batch.n_tokens == batch.n_seqs:
                    n_splits, split_keys = self._latent_split_policy(batch.n_seqs * -(-H // 32), batch.max_seq_len)
                if n_splits > 1:
                    floats = int(lib.llm_latent_attention_scratch_floats(c_int(batch.n_tokens), c_int(H), c_int(kv_rank), c_int(n_splits)))
                    scratch = batch.ws.get("latent.splits", (floats,), torch.float32)
                self._check(lib.llm_latent_attention_mma(
                    _ptr(ql), _ptr(cache), _ptr(batch.seq_start), _ptr(batch.seq_ntok), _ptr(batch.seq_qoff), _ptr(block_table),
                    c_int(block_table.shape[1]), _ptr(out), c_int(batch.n_seqs), c_int(batch.n_tokens), c_int(batch.max_new_tokens),
                    c_int(H), c_int(kv_rank), c_int(Dk - kv_rank), c_int(cache.shape[2]), c_float(scale), c_int(window),
                    c_int(n_splits), c_int(split_keys), _ptr(scratch), _stream()), lib)
                if n_splits > 1:
                    self.launches += 1  # the kernel that merges the splits
                return out
        lib = self.lib()
        self._check(lib.llm_latent_attention_simt(_ptr(ql), _ptr(cache), c_int(dtype_code(ql.dtype)), _ptr(batch.positions),
                                                  _ptr(batch.token_seq), _ptr(block_table), c_int(block_table.shape[1]), _ptr(out),
                                                  c_int(batch.n_tokens), c_int(H), c_int(kv_rank), c_int(Dk - kv_rank),
                                                  c_int(cache.shape[2]), c_float(scale), c_int(window), _stream()), lib)
        return out

    LATENT_TARGET_CTAS = 296  # two CTAs of the latent attention kernel on each of the 148 SMs
    LATENT_MIN_SPLIT_KEYS = 64

    def _latent_split_policy(self, ctas: int, max_seq_len: int):
        """-> (number of key splits, keys per split) of a step of single tokens whose latent attention would run as
        `ctas` CTAs without a split: the key range is cut (at absolute multiples of 64) until about LATENT_TARGET_CTAS
        CTAs stream the cache, but into pieces of at least LATENT_MIN_SPLIT_KEYS keys."""
        want = min(128, self.LATENT_TARGET_CTAS // max(ctas, 1), max_seq_len // self.LATENT_MIN_SPLIT_KEYS)
        if want <= 1:
            return 1, 256
        split_keys = -(-(-(-max_seq_len // want)) // 64) * 64
        return -(-max_seq_len // split_keys), split_keys

    def latent_attention_kernel(self, heads: int, kv_rank: int, rot_dim: int, page: int) -> str:
        """What latent attention of this geometry runs on in bfloat16: "tensor cores" or "CUDA cores"."""
        if self.tensor_cores and self.latent_tensor_cores and self.lib("tensorcore").llm_latent_attention_mma_supported(
                c_int(heads), c_int(kv_rank), c_int(rot_dim)):
            return "tensor cores"
        return "CUDA cores"

    def sigmoid_gate(self, x: torch.Tensor, gate: torch.Tensor, gate_off: int) -> torch.Tensor:
        """x[t, j] *= sigmoid(sum_p gate[p, t, gate_off + j]); gate float32 partial sums [p, n, width]."""
        _need(x, "sigmoid_gate.x"); _need(gate, "sigmoid_gate.gate", torch.float32)
        n, cols = x.shape
        assert gate.is_contiguous() and gate.dim() == 3 and gate.shape[1] >= n
        lib = self.lib()
        self._check(lib.llm_sigmoid_gate(_ptr(x), c_longlong(x.stride(0)), _ptr(gate), c_int(gate.shape[0]), c_longlong(gate.stride(0)),
                                         c_int(gate.shape[2]), c_int(gate_off), c_int(n), c_int(cols), c_int(dtype_code(x.dtype)),
                                         _stream()), lib)
        return x

    # ------------------------------------------------------------------ routed feed-forward
    def route(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], top: int, idx: torch.Tensor,
              share: torch.Tensor) -> None:
        """Per token: logits = w x + bias in float32, idx [n, top] (int32) = the experts with the largest logits (the lower
        index wins a tie), share [n, top] (float32) = the softmax over the chosen logits."""
        _need(x, "route.x"); _need(w, "route.w", x.dtype); _need(idx, "route.idx", torch.int32); _need(share, "route.share", torch.float32)
        n, D = x.shape
        E = w.shape[0]
        assert w.is_contiguous() and w.shape[1] == D and idx.is_contiguous() and share.is_contiguous()
        assert idx.shape == (n, top) and share.shape == (n, top)
        if bias is not None:
            _need(bias, "route.bias", torch.float32)
            assert bias.numel() == E
        lib = self.lib()
        self._check(lib.llm_route(_ptr(x), c_longlong(x.stride(0)), _ptr(w), _ptr(bias), c_int(n), c_int(D), c_int(E), c_int(top),
                                  _ptr(idx), _ptr(share), c_int(dtype_code(x.dtype)), _stream()), lib)

    ROUTED_EPILOGUES = {"gelu": 0, "share": 1, "silu_pairs": 2, "gated_pairs": 2}

    def route_grouped(self, x: torch.Tensor, w: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int, keep: int,
                      norm_eps: float, idx: torch.Tensor, share: torch.Tensor, score: str = "softmax", group_top: int = 1,
                      normalize: bool = True, weight_scale: float = 1.0, gate_out: Optional[torch.Tensor] = None) -> None:
        """Per token: s = softmax(w x) over all experts, or (score "sigmoid") the sigmoid of every logit (float32); choice = s +
        correction; only experts of the `keep` of `groups` equal groups of neighbours with the largest group scores can be chosen
        (a group's score: its largest choice score, or with group_top 2 the sum of its two largest; the others count as minus
        infinity); idx [n, top] = the largest choice scores among them (the lower index wins a tie); share [n, top] = their s
        divided by (the sum of the chosen s + norm_eps), or as they are (normalize False), then times weight_scale. With gate_out
        (float32 [n]) w holds one more row behind the experts' rows and gate_out[t] = sigmoid(that row . x[t]) in float32."""
        _need(x, "route.x"); _need(w, "route.w", x.dtype); _need(idx, "route.idx", torch.int32); _need(share, "route.share", torch.float32)
        n, D = x.shape
        E = w.shape[0] - (1 if gate_out is not None else 0)
        if gate_out is not None:
            _need(gate_out, "route.gate_out", torch.float32)
            assert gate_out.is_contiguous() and gate_out.numel() >= n
        assert w.is_contiguous() and w.shape[1] == D and idx.is_contiguous() and share.is_contiguous()
        assert idx.shape == (n, top) and share.shape == (n, top)
        if correction is not None:
            _need(correction, "route.correction", torch.float32)
            assert correction.numel() == E
        lib = self.lib()
        self._check(lib.llm_route_grouped(_ptr(x), c_longlong(x.stride(0)), _ptr(w), _ptr(correction), c_int(n), c_int(D), c_int(E),
                                          c_int(top), c_int(groups), c_int(keep), c_float(norm_eps), _ptr(idx), _ptr(share),
                                          c_int(dtype_code(x.dtype)), c_int({"softmax": 0, "sigmoid": 1}[score]), c_int(group_top),
                                          c_int(1 if normalize else 0), c_float(weight_scale), _ptr(gate_out), _stream()), lib)

    def routed_tile_rows(self, n_tokens: int = 0, dtype: Optional[torch.dtype] = None, inner=(), per_expert: float = 0.0) -> int:
        """Rows of a tile of the per-expert products: the tensor-core kernel's in bfloat16 when every product's inner
        size (`inner`) is a multiple of 8 (64, or 128 when an expert gets about that many rows: `per_expert`), else the
        CUDA-core kernel's."""
        if dtype == torch.bfloat16 and self.tensor_cores and self.routed_tensor_cores and inner and all(k % 8 == 0 for k in inner):
            return int(self.lib("tensorcore").llm_routed_product_mma_rows(c_int(int(per_expert))))
        return int(self.lib().llm_routed_product_rows())

    def routed_group(self, idx: torch.Tensor, experts: int, tile: int, ws, tag: str, real_experts: Optional[int] = None):
        """Sorts the step's (token, choice) pairs by expert into tiles of `tile` rows -> (tile_expert [tiles] with -1 for
        unused tiles, tile_rows [tiles, tile] with -1 for padding); a pair is token * top + choice. Pairs of experts from
        real_experts on (experts without matrices, dealt with by routed_combine) enter no tile."""
        _need(idx, "routed_group.idx", torch.int32)
        lib = self.lib()
        pairs = idx.numel()
        tiles = int(lib.llm_routed_tiles(c_int(pairs), c_int(experts), c_int(tile)))
        tile_expert = ws.get(tag + ".tile_expert", (tiles,), torch.int32)
        tile_rows = ws.get(tag + ".tile_rows", (tiles, tile), torch.int32)
        self._check(lib.llm_routed_group(_ptr(idx), c_int(pairs), c_int(experts), c_int(tile), c_int(tiles), _ptr(tile_expert),
                                         _ptr(tile_rows), c_int(experts if real_experts is None else real_experts), _stream()), lib)
        return tile_expert, tile_rows

    def routed_product(self, a: torch.Tensor, a_div: int, w: torch.Tensor, tile_expert: torch.Tensor, tile_rows: torch.Tensor,
                       out: torch.Tensor, epilogue: str, share: Optional[torch.Tensor] = None, act="silu") -> torch.Tensor:
        """For every pair p of every tile (expert e): out[p, :] = epi(w[e] a[p // a_div, :]); w [E, N, K]. epilogue "gelu":
        the exact (erf) gelu; "share": times share[p] (float32, flat); "silu_pairs": w holds a gate row and its up row in turn
        ([E, 2 F, K]) and out[p, f] = silu(gate_f) * up_f ([pairs, F]); "gated_pairs": the same rows with the activation `act`
        of a gated feed-forward (ACTIVATIONS; ("clamped_swish", limit, slope) limits both sides)."""
        _need(a, "routed_product.a"); _need(w, "routed_product.w", a.dtype); _need(out, "routed_product.out")
        E, N, K = w.shape
        pairs = epilogue in ("silu_pairs", "gated_pairs")
        assert w.is_contiguous() and a.shape[1] == K and out.shape[1] == (N // 2 if pairs else N)
        assert not pairs or N % 2 == 0
        act_args = self._act_args(act if epilogue == "gated_pairs" else "silu")
        if epilogue == "share":
            _need(share, "routed_product.share", torch.float32)
        if a.dtype == torch.bfloat16 and self.tensor_cores and tile_rows.shape[1] != self.routed_tile_rows():
            lib = self.lib("tensorcore")  # tiles made for the tensor-core kernel (64 or 128 rows)
            assert out.dtype == (torch.float32 if epilogue == "share" else torch.bfloat16)
            self._check(lib.llm_routed_product_mma(_ptr(a), c_longlong(a.stride(0)), c_int(a_div), _ptr(w), c_int(N), c_int(K),
                                                   _ptr(tile_expert), _ptr(tile_rows), c_int(tile_expert.numel()),
                                                   c_int(tile_rows.shape[1]), _ptr(out),
                                                   c_longlong(out.stride(0)), c_int(self.ROUTED_EPILOGUES[epilogue]), _ptr(share),
                                                   *act_args, _stream()), lib)
            return out
        assert tile_rows.shape[1] == self.routed_tile_rows()
        lib = self.lib()
        self._check(lib.llm_routed_product(_ptr(a), c_longlong(a.stride(0)), c_int(a_div), _ptr(w), c_int(N), c_int(K), _ptr(tile_expert),
                                           _ptr(tile_rows), c_int(tile_expert.numel()), _ptr(out), c_longlong(out.stride(0)),
                                           c_int(self.ROUTED_EPILOGUES[epilogue]), _ptr(share), c_int(dtype_code(a.dtype)),
                                           c_int(dtype_code(out.dtype)), *act_args, _stream()), lib)
        return out

    def routed_combine(self, y: torch.Tensor, out: torch.Tensor, top: int, identity=None, extra: Optional[torch.Tensor] = None,
                       extra_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out[t, :] = sum_k y[t * top + k, :] in index order; float32. identity = (idx [n, top] int32, share [n, top] float32,
        real_experts, x [n, D]): a choice whose expert is real_experts or higher is an identity expert and adds share[t, k] * x[t]
        in place of its row of y (which nobody wrote). extra: float32 sums [n, D] or [parts, n, D] added behind the chosen ones
        (an expert that every token uses), times extra_gate[t] (float32 [n]) if given."""
        _need(y, "routed_combine.y", torch.float32); _need(out, "routed_combine.out", torch.float32)
        n, D = out.shape
        assert y.is_contiguous() and out.is_contiguous() and y.shape == (n * top, D)
        id_args = [c_void_p(0), c_void_p(0), c_int(0), c_void_p(0), c_longlong(0), c_int(F32)]
        if identity is not None:
            idx, share, real, x = identity
            _need(idx, "routed_combine.idx", torch.int32); _need(share, "routed_combine.share", torch.float32); _need(x, "routed_combine.x")
            assert idx.is_contiguous() and share.is_contiguous() and idx.shape == (n, top) and share.shape == (n, top) and x.shape[0] >= n and x.shape[1] == D
            id_args = [_ptr(idx), _ptr(share), c_int(real), _ptr(x), c_longlong(x.stride(0)), c_int(dtype_code(x.dtype))]
        ex_args = [c_void_p(0), c_int(0), c_longlong(0), c_void_p(0)]
        if extra is not None:
            _need(extra, "routed_combine.extra", torch.float32)
            assert extra.is_contiguous() and extra.shape[-1] == D and extra.shape[-2] == n
            if extra_gate is not None:
                _need(extra_gate, "routed_combine.gate", torch.float32)
                assert extra_gate.is_contiguous() and extra_gate.numel() >= n
            ex_args = [_ptr(extra), c_int(extra.shape[0] if extra.dim() == 3 else 1), c_longlong(extra.stride(0) if extra.dim() == 3 else 0),
                       _ptr(extra_gate)]
        lib = self.lib()
        self._check(lib.llm_routed_combine(_ptr(y), _ptr(out), c_int(n), c_int(top), c_int(D), *id_args, *ex_args, _stream()), lib)
        return out

    # ------------------------------------------------------------------ norms on a sub-layer's output
    def norm_add(self, h: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor], weight: torch.Tensor, layer_scale: Optional[torch.Tensor],
                 eps: float, copy: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> torch.Tensor:
        """y = a (+ b): float32 [n, dim] or [parts, n, dim] partial sums added in index order; h[:n] += ((y / rms(y)) * weight) *
        layer_scale (eps inside the root; layer_scale optional); copy[:n] (optional, float32 or bfloat16) = the new h."""
        _need(h, "norm_add.h", torch.float32); _need(weight, "norm_add.weight", torch.float32)
        n = h.shape[0] if n_rows is None else n_rows
        dim = h.shape[-1]
        args = []
        for t, name in ((a, "a"), (b, "b")):
            if t is None:
                args += [c_void_p(0), c_int(0), c_longlong(0)]
                continue
            _need(t, "norm_add." + name, torch.float32)
            assert t.is_contiguous() and t.shape[-1] == dim and t.shape[-2] == h.shape[0], "the sums must have the stream's shape"
            args += [_ptr(t), c_int(t.shape[0] if t.dim() == 3 else 1), c_longlong(t.stride(0) if t.dim() == 3 else 0)]
        if layer_scale is not None:
            _need(layer_scale, "norm_add.layer_scale", torch.float32)
            assert layer_scale.numel() == dim
        code = F32
        if copy is not None:
            _need(copy, "norm_add.copy")
            assert copy.is_contiguous() and copy.shape[-1] == dim and copy.shape[0] >= n
            code = dtype_code(copy.dtype)
        assert h.is_contiguous() and weight.numel() == dim and a is not None
        lib = self.lib()
        self._check(lib.llm_norm_add(_ptr(h), *args, _ptr(weight), _ptr(layer_scale), c_float(eps), _ptr(copy), c_int(code), c_int(n),
                                     c_int(dim), _stream()), lib)
        return h

    # ------------------------------------------------------------------ gated attention
    def qkv_prep(self, parts: torch.Tensor, heads: int, kv_heads: int, dk: int, dv: int, q_norm: Optional[torch.Tensor],
                 k_norm: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], batch,
                 block_table: torch.Tensor, q_out: torch.Tensor, kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
                 mix_role: int = 0, mix_weight: Optional[torch.Tensor] = None, v_first: Optional[torch.Tensor] = None,
                 norm_wide: bool = False) -> None:
        """From the float32 sums `parts` [p, n, width] of a product whose columns begin with [q: heads * dk | k: kv_heads * dk |
        v: kv_heads * dv] (kv_heads 0: queries alone, nothing to write): RMS norm of every query and key head with the weights
        q_norm / k_norm [dk] (None: no norm), or with norm_wide ONE RMS norm over all query heads' numbers together with q_norm
        [heads * dk] and one over all key heads' with k_norm [kv_heads * dk]; rotation
        of the first 2 * cos.shape[1] numbers of each head (half-split pairs) at the token's position, q into q_out
        [n, heads * dk], k and v into the token's page of kcache [pages, kv_heads, page, dk] / vcache [.., dv] (None: no write).
        mix_role 1: the values are also left in v_first (float32 [n, kv_heads * dv]); 2: v <- (1 - m) v + m v_first before
        the write, m = mix_weight (a float32 scalar on the device)."""
        _need(parts, "qkv_prep.parts", torch.float32); _need(q_out, "qkv_prep.q")
        assert parts.dim() == 3 and parts.is_contiguous()
        n = batch.n_tokens
        rot_dims = 0 if cos is None else 2 * cos.shape[1]
        for t, name in ((q_norm, "q_norm"), (k_norm, "k_norm"), (cos, "cos"), (sin, "sin"), (mix_weight, "mix_weight"), (v_first, "v_first")):
            if t is not None:
                _need(t, "qkv_prep." + name, torch.float32)
                assert t.is_contiguous()
        wide = (heads, kv_heads) if norm_wide else (1, 1)
        assert (q_norm is None or q_norm.numel() == wide[0] * dk) and (k_norm is None or kv_heads == 0 or k_norm.numel() == wide[1] * dk)
        page = 1
        if kcache is not None:
            _need(kcache, "qkv_prep.kcache", q_out.dtype); _need(vcache, "qkv_prep.vcache", q_out.dtype)
            assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[1] == kv_heads and kcache.shape[3] == dk
            assert vcache.shape[:3] == kcache.shape[:3] and vcache.shape[3] == dv
            page = kcache.shape[2]
        if v_first is not None:
            assert v_first.shape[0] >= n and v_first.shape[1] == kv_heads * dv
        lib = self.lib()
        self._check(lib.llm_qkv_prep(_ptr(parts), c_int(parts.shape[0]), c_longlong(parts.stride(0)), c_int(parts.shape[2]), c_int(heads),
                                     c_int(kv_heads), c_int(dk), c_int(dv), c_int(rot_dims), _ptr(q_norm), _ptr(k_norm), c_float(eps),
                                     _ptr(cos), _ptr(sin), _ptr(batch.positions), _ptr(batch.token_seq), _ptr(block_table),
                                     c_int(block_table.shape[1]), _ptr(q_out), c_longlong(q_out.stride(0)), _ptr(kcache), _ptr(vcache),
                                     c_int(page), c_int(mix_role), _ptr(mix_weight), _ptr(v_first), c_int(dtype_code(q_out.dtype)),
                                     c_int(n), c_int(1 if norm_wide else 0), _stream()), lib)

    def gated_attention(self, q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, batch, block_table: torch.Tensor,
                        out: torch.Tensor, nq: int, nkv: int, dk: int, dv: int, scale: float, window: int = 0, chunk: int = 0,
                        sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, gate_off: int = 0,
                        gate_per_head: bool = False) -> torch.Tensor:
        """Causal attention of every token of the step over the cache positions of its request from the later of the window's
        and the chunk's start (chunks are [c * chunk, (c + 1) * chunk) in absolute positions; 0: none) up to its own; keys of dk
        and values of dv numbers a head; sink (float32 [nq], optional): exp(sink[head]) is one more term of the softmax's
        denominator; gate (float32 partial sums [p, n, width], optional): the result times sigmoid(sum_p gate[p, t, gate_off +
        head * dv + d]), or with gate_per_head one gate a head at column gate_off + head. q rows of [nq * dk]; out [n, nq * dv]."""
        _need(q, "attention.q"); _need(kcache, "attention.kcache", q.dtype); _need(vcache, "attention.vcache", q.dtype)
        _need(out, "attention.out", q.dtype); _need(block_table, "attention.block_table", torch.int32)
        assert kcache.is_contiguous() and vcache.is_contiguous() and block_table.is_contiguous()
        assert kcache.shape[1] == nkv and kcache.shape[3] == dk and vcache.shape[3] == dv
        if sink is not None:
            _need(sink, "attention.sink", torch.float32)
            assert sink.numel() == nq and sink.is_contiguous()
        gp, gs, gw = 0, 0, 0
        if gate is not None:
            _need(gate, "attention.gate", torch.float32)
            assert gate.dim() == 3 and gate.is_contiguous()
            gp, gs, gw = gate.shape[0], gate.stride(0), gate.shape[2]
        page = kcache.shape[2]
        if q.dtype == torch.bfloat16 and self.tensor_cores and self.gated_attention_tensor_cores:
            lib = self.lib("tensorcore")
            if lib.llm_gated_attention_mma_supported(c_int(nq), c_int(nkv), c_int(dk), c_int(dv), c_longlong(q.stride(0)), c_longlong(out.stride(0))):
                n_splits, split_keys, scratch = 1, 256, None
                if batch.max_new_tokens == 1 and batch.n_tokens == batch.n_seqs and dk == dv:
                    # single decoded tokens: the keys a token may see (its chunk at most) in pieces side by side
                    reach = min(batch.max_seq_len, chunk) if chunk > 0 else batch.max_seq_len
                    n_splits, split_keys = self._split_policy(batch.n_seqs * nkv, reach, dk)
                    if n_splits > 1:
                        floats = int(lib.llm_attention_mma_scratch_floats(c_int(batch.n_tokens), c_int(nq), c_int(dv), c_int(n_splits)))
                        scratch = batch.ws.get("attention.splits", (floats,), torch.float32)
                self._check(lib.llm_gated_attention_mma(
                    _ptr(q), c_longlong(q.stride(0)), _ptr(kcache), _ptr(vcache), _ptr(batch.seq_start), _ptr(batch.seq_ntok), _ptr(batch.seq_qoff),
                    _ptr(block_table), c_int(block_table.shape[1]), _ptr(out), c_longlong(out.stride(0)), c_int(batch.n_seqs),
                    c_int(batch.max_new_tokens), c_int(nq), c_int(nkv), c_int(dk), c_int(dv), c_int(page), c_float(scale), c_int(window),
                    c_int(chunk), _ptr(sink), _ptr(gate), c_int(gp), c_longlong(gs), c_int(gw), c_int(gate_off), c_int(1 if gate_per_head else 0),
                    c_int(batch.n_tokens), c_int(n_splits), c_int(split_keys), _ptr(scratch), _stream()), lib)
                if n_splits > 1:
                    self.launches += 1  # the kernel that merges the pieces
                return out
        lib = self.lib()
        self._check(lib.llm_gated_attention_simt(_ptr(q), c_longlong(q.stride(0)), _ptr(kcache), _ptr(vcache), c_int(dtype_code(q.dtype)),
                                                 _ptr(batch.positions), _ptr(batch.token_seq), _ptr(block_table),
                                                 c_int(block_table.shape[1]), _ptr(out), c_longlong(out.stride(0)), c_int(batch.n_tokens),
                                                 c_int(nq), c_int(nkv), c_int(dk), c_int(dv), c_int(page), c_float(scale), c_int(window),
                                                 c_int(chunk), _ptr(sink), _ptr(gate), c_int(gp), c_longlong(gs), c_int(gw), c_int(gate_off),
                                                 c_int(1 if gate_per_head else 0), _stream()), lib)
        return out

    def gated_attention_kernel(self, nq: int, nkv: int, dk: int, dv: int) -> str:
        """What a bfloat16 model's gated attention of this geometry runs on: "tensor cores" or "CUDA cores"."""
        if self.tensor_cores and self.gated_attention_tensor_cores:
            lib = self.lib("tensorcore")
            if lib.llm_gated_attention_mma_supported(c_int(nq), c_int(nkv), c_int(dk), c_int(dv), c_longlong(nq * dk), c_longlong(nq * dv)):
                return "tensor cores"
        return "CUDA cores"

    # ------------------------------------------------------------------ selective scan
    def conv_silu(self, parts: torch.Tensor, x_off: int, channels: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                  conv_state: torch.Tensor, batch, out: torch.Tensor) -> torch.Tensor:
        """out[t, c] = silu(bias[c] + sum_j weight[c, j] * x[t - (K - 1) + j, c]) over each request's own tokens, x = columns
        x_off .. x_off + channels of the float32 sums `parts` [p, n, width]; inputs before the step's portion come from
        conv_state [slots, K - 1, channels] (float32) at the request's slot, which afterwards holds the request's last K - 1
        inputs."""
        _need(parts, "conv.parts", torch.float32); _need(weight, "conv.weight", out.dtype); _need(conv_state, "conv.state", torch.float32)
        _need(out, "conv.out")
        K = weight.shape[1]
        n = batch.n_tokens
        assert parts.dim() == 3 and parts.is_contiguous() and weight.is_contiguous() and weight.shape[0] == channels
        assert conv_state.is_contiguous() and tuple(conv_state.shape[1:]) == (K - 1, channels)
        assert out.is_contiguous() and out.shape[0] >= n and out.shape[1] == channels
        if bias is not None:
            _need(bias, "conv.bias", torch.float32)
            assert bias.numel() == channels
        lib = self.lib()
        self._check(lib.llm_conv_silu(_ptr(parts), c_int(parts.shape[0]), c_longlong(parts.stride(0)), c_int(parts.shape[2]), c_int(x_off),
                                      c_int(channels), c_int(K), _ptr(weight), _ptr(bias), _ptr(conv_state), _ptr(batch.token_seq),
                                      _ptr(batch.seq_qoff), _ptr(batch.seq_ntok), _ptr(batch.seq_slot), _ptr(out),
                                      c_int(dtype_code(out.dtype)), c_int(n), c_int(batch.n_seqs), _stream()), lib)
        if K > 1:
            self.launches += 1  # the kernel that renews the slot
        return out

    def dt_softplus(self, proj: torch.Tensor, rank: int, weight_t: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                    n_tokens: int) -> torch.Tensor:
        """out[t, c] (float32) = softplus(bias[c] + sum_r weight_t[r, c] * proj[t, r]) for the first `rank` columns of the
        float32 rows proj; weight_t [rank, channels] is the map stored transposed."""
        _need(proj, "dt.proj", torch.float32); _need(weight_t, "dt.weight"); _need(out, "dt.out", torch.float32)
        C = weight_t.shape[1]
        assert weight_t.is_contiguous() and weight_t.shape[0] == rank and out.is_contiguous() and out.shape[1] == C and out.shape[0] >= n_tokens
        if bias is not None:
            _need(bias, "dt.bias", torch.float32)
            assert bias.numel() == C
        lib = self.lib()
        self._check(lib.llm_dt_softplus(_ptr(proj), c_longlong(proj.stride(0)), c_int(rank), _ptr(weight_t), _ptr(bias), c_int(C), _ptr(out),
                                        c_int(dtype_code(weight_t.dtype)), c_int(n_tokens), _stream()), lib)
        return out

    def selective_scan(self, xc: torch.Tensor, dt: torch.Tensor, proj: torch.Tensor, b_off: int, c_off: int, state_size: int,
                       zparts: torch.Tensor, z_off: int, a_log: torch.Tensor, skip: Optional[torch.Tensor], state: torch.Tensor, batch,
                       out: torch.Tensor, dt_bias: Optional[torch.Tensor] = None, dt_raw: bool = False) -> torch.Tensor:
        """Token after token of every request: S[c, n] <- exp(dt[t, c] * A[c, n]) * S[c, n] + dt[t, c] * xc[t, c] * B[t, n],
        y[t, c] = sum_n S[c, n] * C[t, n] + skip[c] * xc[t, c], out[t, c] = y * silu(z[t, c]); A = -exp(a_log) [channels, N];
        B, C = columns b_off.., c_off.. of the float32 rows proj; z = columns z_off.. of the float32 sums zparts [p, n, width];
        state [slots, channels, N] float32, read from and written to the request's slot. dt_raw: dt holds the sums of the step-size
        product, and the kernel applies softplus(dt + dt_bias) itself."""
        _need(xc, "scan.x"); _need(dt, "scan.dt", torch.float32); _need(proj, "scan.proj", torch.float32)
        _need(zparts, "scan.z", torch.float32); _need(a_log, "scan.a_log", torch.float32); _need(state, "scan.state", torch.float32)
        _need(out, "scan.out", xc.dtype)
        C, N = a_log.shape
        assert N == state_size and xc.is_contiguous() and dt.is_contiguous() and out.is_contiguous() and a_log.is_contiguous()
        assert xc.shape[1] == C and dt.shape[1] == C and out.shape[1] == C and state.is_contiguous() and tuple(state.shape[1:]) == (C, N)
        assert zparts.dim() == 3 and zparts.is_contiguous()
        if skip is not None:
            _need(skip, "scan.skip", torch.float32)
            assert skip.numel() == C
        lib = self.lib()
        # a long portion is cut into pieces that run side by side (two passes and a carry between them); short ones and single
        # decoded tokens are walked in one pass
        piece = int(lib.llm_selective_scan_piece())
        pieces, piece_state, piece_sumdt = 0, None, None
        if batch.max_new_tokens >= self.SCAN_PIECES_FROM:
            pieces = batch.n_tokens // piece + batch.n_seqs
            piece_state = batch.ws.get("scan.piece_state", (pieces, C, N), torch.float32)
            piece_sumdt = batch.ws.get("scan.piece_sumdt", (pieces, C), torch.float32)
        self._check(lib.llm_selective_scan(_ptr(xc), _ptr(dt), _ptr(proj), c_longlong(proj.stride(0)), c_int(b_off), c_int(c_off),
                                           _ptr(zparts), c_int(zparts.shape[0]), c_longlong(zparts.stride(0)), c_int(zparts.shape[2]),
                                           c_int(z_off), _ptr(a_log), _ptr(skip), _ptr(state), _ptr(batch.seq_qoff), _ptr(batch.seq_ntok),
                                           _ptr(batch.seq_slot), c_int(C), c_int(N), _ptr(out), c_int(dtype_code(xc.dtype)),
                                           c_int(batch.n_seqs), c_int(batch.max_new_tokens), c_int(pieces), _ptr(piece_state),
                                           _ptr(piece_sumdt), _ptr(dt_bias), c_int(1 if dt_raw else 0), _stream()), lib)
        if pieces:
            self.launches += 2
        return out

    SCAN_PIECES_FROM = 192  # tokens of the step's longest portion from which the scan runs in pieces

    LOWRANK_OUT = {"softplus": 0, "sigmoid_root": 1, "exp_neg_exp": 2}

    def lowrank_map(self, proj: torch.Tensor, rank: int, weight_t: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                    n_tokens: int, in_act: Optional[str] = None, out_act: str = "softplus", param: float = 0.0) -> torch.Tensor:
        """out[t, c] (float32) = g(bias[c] + sum_r weight_t[r, c] * f(proj[t, r])) for the first `rank` columns of the float32 rows
        proj; weight_t [rank, channels]. f: None or "tanh". g: "softplus"; "sigmoid_root": sigmoid(z)^(1 / param); "exp_neg_exp":
        exp(-exp(z)). dt_softplus is this map with f None and g softplus."""
        _need(proj, "lowrank.proj", torch.float32); _need(weight_t, "lowrank.weight"); _need(out, "lowrank.out", torch.float32)
        C = weight_t.shape[1]
        assert weight_t.is_contiguous() and weight_t.shape[0] == rank and out.is_contiguous() and out.shape[1] == C and out.shape[0] >= n_tokens
        assert in_act in (None, "tanh")
        if bias is not None:
            _need(bias, "lowrank.bias", torch.float32)
            assert bias.numel() == C
        lib = self.lib()
        self._check(lib.llm_lowrank_map(_ptr(proj), c_longlong(proj.stride(0)), c_int(rank), _ptr(weight_t), _ptr(bias), c_int(C), _ptr(out),
                                        c_int(dtype_code(weight_t.dtype)), c_int(n_tokens), c_int(1 if in_act == "tanh" else 0),
                                        c_int(self.LOWRANK_OUT[out_act]), c_float(param), _stream()), lib)
        return out

    # ------------------------------------------------------------------ two branches into one
    def pair_combine(self, a: torch.Tensor, b: torch.Tensor, wa: Optional[torch.Tensor], wb: Optional[torch.Tensor], ca: float, cb: float,
                     eps: float, out: torch.Tensor, n_rows: Optional[int] = None) -> torch.Tensor:
        """out[:n] (float32 [n, dim]) = ca * f(a) + cb * f(b) for two sets of float32 sums ([n, dim] or [parts, n, dim], added in index
        order); with a weight (float32 [dim]) f is the row divided by its root mean square (eps inside the root) times the weight,
        without one the identity."""
        n = out.shape[0] if n_rows is None else n_rows
        dim = out.shape[1]
        args = []
        for t, name in ((a, "a"), (b, "b")):
            _need(t, "pair_combine." + name, torch.float32)
            assert t.is_contiguous() and t.shape[-1] == dim and t.shape[-2] >= n
            args += [_ptr(t), c_int(t.shape[0] if t.dim() == 3 else 1), c_longlong(t.stride(0) if t.dim() == 3 else 0)]
        for w in (wa, wb):
            if w is not None:
                _need(w, "pair_combine.weight", torch.float32)
                assert w.numel() == dim
        _need(out, "pair_combine.out", torch.float32)
        assert out.is_contiguous()
        lib = self.lib()
        self._check(lib.llm_pair_combine(*args, _ptr(wa), _ptr(wb), c_float(ca), c_float(cb), c_float(eps), _ptr(out), c_int(n), c_int(dim),
                                         _stream()), lib)
        return out

    # ------------------------------------------------------------------ mixers with a matrix of state per head
    LINEAR_STATE_RULES = {"decay_write_read": 0, "bonus_read_decay_write": 1, "delta": 2}

    def linear_state_shape(self, heads: int, dk: int, dv: int):
        """Shape of the float32 state that linear_state keeps per request (its layout is the kernel's own)."""
        if not 1 <= dk <= 512:
            raise ValueError(f"linear state: a key size of {dk} is beyond the kernel (1..512)")
        lanes = 1  # a column's dk numbers lie on `lanes` lanes of a warp, 16 a lane (llm_linear_state_lanes)
        while lanes * 16 < dk:
            lanes *= 2
        return (heads, lanes * 16, dv)

    @staticmethod
    def _sums(t: torch.Tensor, off: int, name: str):
        """(pointer, parts, stride between parts, row width, column offset) of float32 sums [parts, n, width] or rows [n, width]."""
        _need(t, name, torch.float32)
        assert t.is_contiguous() and t.dim() in (2, 3)
        return [_ptr(t), c_int(t.shape[0] if t.dim() == 3 else 1), c_longlong(t.stride(0) if t.dim() == 3 else 0), c_int(t.shape[-1]), c_int(off)]

    def linear_state(self, rule: str, q, q_off: int, k, k_off: int, v, v_off: int, decay: torch.Tensor, decay_off: int,
                     bonus: Optional[torch.Tensor], state: torch.Tensor, batch, out: torch.Tensor, heads: int, kv_heads: int, dk: int,
                     dv: int, q_scale: float = 1.0, unit_eps: float = -1.0, decay_const: bool = False) -> torch.Tensor:
        """Token after token of every request, per head a matrix S [dk, dv] (float32, in the request's slot of `state`):
        "decay_write_read": S <- diag(a) S + k v^T, o = S^T q; "bonus_read_decay_write": o = (S + diag(bonus) k v^T)^T q, then
        S <- diag(a) S + k v^T; "delta": S <- g S, w = beta (v - S^T k), S <- S + k w^T, o = S^T q with q and k made unit vectors
        per head first (x / sqrt(sum x^2 + unit_eps); unit_eps < 0: as they are). q is multiplied by q_scale. q, k, v: float32 sums
        ([parts, n, width] or [n, width]) read at column offsets, q and k with kv_heads heads of dk (head h reads head
        h // (heads / kv_heads)), v with heads of dv. decay: float32 rows; at decay_off a number per (head, key channel), or for
        "delta" [g: heads | beta: heads]; with decay_const a single row that holds for every token (decays that are constants
        of the model). out float32 [n, heads * dv]."""
        _need(decay, "linear_state.decay", torch.float32); _need(state, "linear_state.state", torch.float32); _need(out, "linear_state.out", torch.float32)
        assert decay.is_contiguous() and decay.dim() == 2 and state.is_contiguous() and out.is_contiguous() and out.shape[1] == heads * dv
        assert tuple(state.shape[1:]) == tuple(self.linear_state_shape(heads, dk, dv))
        if bonus is not None:
            _need(bonus, "linear_state.bonus", torch.float32)
            assert bonus.is_contiguous() and bonus.numel() == heads * dk
        lib = self.lib()
        self._check(lib.llm_linear_state(c_int(self.LINEAR_STATE_RULES[rule]), *self._sums(q, q_off, "linear_state.q"),
                                         *self._sums(k, k_off, "linear_state.k"), *self._sums(v, v_off, "linear_state.v"), _ptr(decay),
                                         c_int(decay.shape[1]), c_int(decay_off), _ptr(bonus), _ptr(state), _ptr(batch.seq_qoff),
                                         _ptr(batch.seq_ntok), _ptr(batch.seq_slot), _ptr(out), c_int(batch.n_tokens), c_int(batch.n_seqs), c_int(heads),
                                         c_int(kv_heads), c_int(dk), c_int(dv), c_float(q_scale), c_float(unit_eps), c_int(1 if decay_const else 0),
                                         _stream()), lib)
        return out

    def rotate_sums(self, x, x_off: int, heads: int, dk: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                    out: torch.Tensor, n_tokens: int, scaled_from: Optional[int] = None, scale: float = 1.0) -> torch.Tensor:
        """out[t] (float32 [n, heads * dk]) = the `heads` heads of dk numbers that lie side by side from column x_off of the float32
        sums x, the first 2 * cos.shape[1] numbers of every head rotated (half-split pairs) at the token's position; heads from
        `scaled_from` on are then multiplied by `scale`. Nothing is rounded: for mixers whose recurrence reads rotated queries and keys."""
        _need(out, "rotate_sums.out", torch.float32); _need(positions, "rotate_sums.positions", torch.int32)
        assert out.is_contiguous() and out.shape[1] == heads * dk and out.shape[0] >= n_tokens
        rot = 0 if cos is None else 2 * cos.shape[1]
        for t in (cos, sin):
            if t is not None:
                _need(t, "rotate_sums.table", torch.float32)
                assert t.is_contiguous()
        lib = self.lib()
        self._check(lib.llm_rotate_sums(*self._sums(x, x_off, "rotate_sums.x"), c_int(heads), c_int(dk), c_int(rot), _ptr(cos), _ptr(sin),
                                        _ptr(positions), _ptr(out), c_int(n_tokens), c_int(heads if scaled_from is None else scaled_from),
                                        c_float(scale), _stream()), lib)
        return out

    def token_shift(self, x: torch.Tensor, mu: torch.Tensor, shift_state: torch.Tensor, batch, out: torch.Tensor) -> torch.Tensor:
        """out[s, t] = x[t] + (x[t - 1] - x[t]) * mu[s] for every blend s (mu float32 [blends, dim]), t - 1 the request's token before t:
        of this step, or for a portion's first token the row kept in shift_state [slots, dim] (float32), which afterwards holds the
        request's last row."""
        _need(x, "token_shift.x"); _need(mu, "token_shift.mu", torch.float32); _need(shift_state, "token_shift.state", torch.float32)
        _need(out, "token_shift.out", x.dtype)
        n, D = batch.n_tokens, x.shape[1]
        assert x.is_contiguous() and mu.is_contiguous() and mu.shape[1] == D and shift_state.is_contiguous() and shift_state.shape[1] == D
        assert out.is_contiguous() and tuple(out.shape) == (mu.shape[0], n, D) and x.shape[0] >= n
        lib = self.lib()
        self._check(lib.llm_token_shift(_ptr(x), _ptr(mu), c_int(mu.shape[0]), _ptr(shift_state), _ptr(batch.token_seq), _ptr(batch.seq_qoff),
                                        _ptr(batch.seq_ntok), _ptr(batch.seq_slot), _ptr(out), c_int(dtype_code(x.dtype)), c_int(n),
                                        c_int(batch.n_seqs), c_int(D), _stream()), lib)
        self.launches += 1  # the kernel that renews the slot
        return out

    def delta_gates(self, a, a_off: int, b, b_off: int, a_log: torch.Tensor, dt_bias: torch.Tensor, out: torch.Tensor, n_tokens: int) -> torch.Tensor:
        """out[t] (float32 [n, 2 heads]) = [exp(-exp(a_log) * softplus(a[t] + dt_bias)) | sigmoid(b[t])]; a, b: float32 sums read
        at column offsets, a number a head."""
        H = a_log.numel()
        _need(a_log, "delta_gates.a_log", torch.float32); _need(dt_bias, "delta_gates.dt_bias", torch.float32); _need(out, "delta_gates.out", torch.float32)
        assert dt_bias.numel() == H and out.is_contiguous() and out.shape[1] == 2 * H and out.shape[0] >= n_tokens
        lib = self.lib()
        self._check(lib.llm_delta_gates(*self._sums(a, a_off, "delta_gates.a"), *self._sums(b, b_off, "delta_gates.b"), _ptr(a_log),
                                        _ptr(dt_bias), _ptr(out), c_int(n_tokens), c_int(H), _stream()), lib)
        return out

    def head_norm_gate(self, o: torch.Tensor, weight: torch.Tensor, gate, gate_off: int, eps: float, out: torch.Tensor, n_tokens: int,
                       heads: int, dv: int) -> torch.Tensor:
        """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * silu(gate[t, h]) per head of dv numbers; o float32
        [n, heads * dv]; weight float32 [dv] (one for all heads) or [heads * dv]; gate: float32 sums read at gate_off (None: no gate)."""
        _need(o, "head_norm_gate.o", torch.float32); _need(weight, "head_norm_gate.weight", torch.float32); _need(out, "head_norm_gate.out")
        assert o.is_contiguous() and out.is_contiguous() and o.shape[1] == heads * dv and out.shape[1] == heads * dv
        assert weight.numel() in (dv, heads * dv) and weight.is_contiguous()
        g = self._sums(gate, gate_off, "head_norm_gate.gate") if gate is not None else [c_void_p(0), c_int(0), c_longlong(0), c_int(0), c_int(0)]
        lib = self.lib()
        self._check(lib.llm_head_norm_gate(_ptr(o), _ptr(weight), c_int(1 if (weight.numel() == heads * dv and heads > 1) else 0), *g, c_float(eps),
                                           _ptr(out), c_int(dtype_code(out.dtype)), c_int(n_tokens), c_int(heads), c_int(dv), _stream()), lib)
        return out

    # ------------------------------------------------------------------ sampling
    def sample_scratch_words(self, n_rows: int, vocab: int) -> int:
        """4-byte words of scratch that `sample` needs for n_rows rows."""
        return 2 * n_rows * int(self.lib().llm_sample_chunks(c_int(vocab)))

    def sample(self, logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
               seeds: Optional[torch.Tensor] = None, draws: Optional[torch.Tensor] = None,
               n_rows: Optional[int] = None, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out[r] (int32) = greedy or temperature choice for logits row r (float32). scratch: int32
        tensor of sample_scratch_words(rows, vocab) elements (made here when not given)."""
        _need(logits, "sample.logits", torch.float32)
        if not (out.is_cuda or out.is_pinned()) or out.dtype != torch.int32 or not out.is_contiguous():
            raise KernelError("sample.out: expected a contiguous int32 tensor on the device or in pinned host memory")
        n = logits.shape[0] if n_rows is None else n_rows
        for t, nm in ((temperature, "temperature"), (seeds, "seeds"), (draws, "draws")):
            if t is not None:
                _need(t, f"sample.{nm}", torch.float32 if nm == "temperature" else torch.int32)
        lib = self.lib()
        words = self.sample_scratch_words(max(n, 1), logits.shape[1])
        if scratch is None:
            scratch = torch.empty(words, dtype=torch.int32, device=logits.device)
        assert scratch.dtype == torch.int32 and scratch.numel() >= words and scratch.is_cuda
        self._check(lib.llm_sample(_ptr(logits), c_longlong(logits.stride(0)), _ptr(temperature), _ptr(seeds),
                                   _ptr(draws), _ptr(out), c_int(n), c_int(logits.shape[1]), _ptr(scratch), _stream()), lib)
        self.launches += 1  # two kernels
        return out

    def set_dependent_launch(self, on: bool) -> None:
        """Programmatic dependent launch of the kernels (on by default); off for A/B measurements."""
        for name in ("core", "tensorcore"):
            self.lib(name).llm_set_dependent_launch(c_int(1 if on else 0))


_OPS: Optional[CudaOps] = None


def get_ops() -> CudaOps:
    global _OPS
    if _OPS is None:
        _OPS = CudaOps()
    return _OPS
