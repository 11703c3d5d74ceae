"""Typed Python entry points of the CUDA kernels (``csrc/``), called through ctypes.

Each function checks what the kernel cannot check (device, type, contiguity),
passes raw pointers and the current CUDA stream, and turns a refusal of the
launcher into a :class:`KernelError` that names the kernel and the reason.
There is no other implementation behind these names: without the built library
they raise.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_float, c_int, c_long, c_void_p

import torch

from . import library

OUT_STORE = 0        # y (compute type) = x·Wᵀ
OUT_STORE_F32 = 1    # y (fp32) = x·Wᵀ
OUT_ADD_F32 = 2      # y (fp32) += x·Wᵀ
OUT_SWIGLU = 3       # y (compute type) = silu(gate)·up, W's rows alternating gate and up rows (tensor-core kernel only)
OUT_GEGLU = 4        # the same with the tanh form of GELU as the gate's activation
OUT_RELU2 = 5        # y (compute type) = relu(x·Wᵀ + bias)², the activation finished in the product's epilogue
OUT_GELU = 6         # y (compute type) = gelu(x·Wᵀ + bias), the exact form v·Phi(v), finished in the product's epilogue
_GATED = (OUT_SWIGLU, OUT_GEGLU)
_STORES = (OUT_STORE, OUT_RELU2, OUT_GELU)      # the modes whose output has the compute type and the weight's row count

_ERRORS = {
    -1: "unsupported element type",
    -2: "a size is out of the range this kernel takes",
    -3: "the launch failed (see the CUDA error state)",
    -4: "a pointer or pitch is not aligned as the kernel needs",
    -5: "this combination of options is not supported",
    -6: "a CUDA driver call failed",
}


class KernelError(RuntimeError):
    pass


_launches = 0


def launch_count(add: int = 0) -> int:
    """Kernels of this library launched so far in this process (``add`` adjusts it: a graph replay
    adds the kernels it holds)."""
    global _launches
    _launches += add
    return _launches


def _check(name: str, code: int) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise KernelError(f"{name}: {_ERRORS.get(code, f'error {code}')}")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported element type {t.dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream() -> c_void_p:
    """The current CUDA stream of the current device (the capture stream while a graph is recorded).  A launch asks
    for it every time; ``torch.cuda.current_stream()`` costs several microseconds a call, which is a quarter of the
    host time of a short prompt's step, so the raw accessor is used where this torch has it."""
    global _device_index
    if _raw_stream is None:
        return c_void_p(torch.cuda.current_stream().cuda_stream)
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return c_void_p(_raw_stream(_device_index))


def _stream_int() -> int:
    """The same as a plain integer, for the functions whose argument types are declared (see ``lib``)."""
    return _stream().value or 0


def copy_to_device(dst_ptr: int, src_ptr: int, n_bytes: int, done: "Mark | None" = None) -> None:
    """``n_bytes`` from pinned host memory at ``src_ptr`` to device memory at ``dst_ptr`` on the current stream (the
    caller keeps both alive and does not touch the host bytes until the copy is done: ``done.wait()`` tells)."""
    code = lib().llmi_copy_to_device(c_void_p(dst_ptr), c_void_p(src_ptr), c_long(n_bytes),
                                     c_void_p(done.handle if done is not None else 0), _stream())
    if code != 0:
        raise KernelError(f"copy_to_device: {_ERRORS.get(code, f'error {code}')}")


class Mark:
    """A point in a stream's work that the host can wait for (set by :func:`copy_to_device`)."""

    def __init__(self):
        fn = lib().llmi_mark_new
        fn.restype = c_void_p
        self.handle = fn()
        if not self.handle:
            raise KernelError("mark: the device gave none")

    def wait(self) -> None:
        if lib().llmi_mark_wait(c_void_p(self.handle)) != 0:
            raise KernelError("mark: the wait failed")

    def __del__(self):
        try:
            if self.handle:
                lib().llmi_mark_free(c_void_p(self.handle))
                self.handle = None
        except Exception:
            pass


def copy_to_host(dst_ptr: int, src_ptr: int, n_bytes: int) -> None:
    """``n_bytes`` from device memory at ``src_ptr`` to pinned host memory at ``dst_ptr`` on the current stream; returns
    when they are there."""
    code = lib().llmi_copy_to_host(c_void_p(dst_ptr), c_void_p(src_ptr), c_long(n_bytes), _stream())
    if code != 0:
        raise KernelError(f"copy_to_host: {_ERRORS.get(code, f'error {code}')}")


def _addr(t) -> int | None:
    return None if t is None else t.data_ptr()


def _ptr(t) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors only (there is no CPU path)")


_configured = False


def lib():
    global _configured
    l = library.load()
    if not _configured:
        for name in ("llmi_embed", "llmi_rmsnorm", "llmi_swiglu", "llmi_linear_simt", "llmi_rope_store",
                     "llmi_attention_generic", "llmi_argmax", "llmi_sample", "llmi_gemm_tc", "llmi_gemm_tc_splits",
                     "llmi_attention_decode", "llmi_attention_decode_supported", "llmi_attention_decode_resident",
                     "llmi_attention_decode_fused", "llmi_attention_decode_mma", "llmi_attention_decode_mma_supported",
                     "llmi_attention_decode_mma_resident", "llmi_attention_decode_clusters_resident",
                     "llmi_attention_prefill", "llmi_attention_prefill_supported", "llmi_gemm_skinny",
                     "llmi_gemm_skinny_max_tokens", "llmi_attention_prefill_tc", "llmi_attention_prefill_tc_supported",
                     "llmi_sm_count", "llmi_dyt", "llmi_dyt_add", "llmi_stream_add", "llmi_linear_simt_batched",
                     "llmi_latent_prepare", "llmi_latent_q_rotate", "llmi_attention_latent", "llmi_delta_prepare",
                     "llmi_delta_conv_carry", "llmi_delta_recurrence", "llmi_delta_finish", "llmi_moe_route", "llmi_moe_up",
                     "llmi_moe_down", "llmi_moe_grouped", "llmi_linear_heads_mma", "llmi_attention_latent_mma", "llmi_attention_latent_mma_supported",
                     "llmi_conv_add", "llmi_conv_carry", "llmi_qkv_prepare", "llmi_attention_flex", "llmi_diff_combine",
                     "llmi_gdelta_prepare", "llmi_dplr_recurrence", "llmi_activate", "llmi_attention_maps_mma", "llmi_attention_maps_mma_supported", "llmi_tanh_rows", "llmi_norm_conv_token",
                     "llmi_layernorm", "llmi_depth_mix", "llmi_gate_rows", "llmi_pool_rows", "llmi_mix_layernorm",
                     "llmi_moe_identity_add", "llmi_channel_decay", "llmi_rows_activate", "llmi_decay_recurrence",
                     "llmi_normed_pair", "llmi_stream_axpy_norm"):
            getattr(l, name).restype = c_int
        l.llmi_gemm_tc_workspace.restype = c_long
        l.llmi_delta_state_floats.restype = c_long
        l.llmi_attention_latent_mma_workspace.restype = c_long
        l.llmi_attention_maps_mma_workspace.restype = c_long
        l.llmi_moe_group_ints.restype = c_long
        l.llmi_attention_decode_workspace.restype = c_long
        # The launchers of a prompt's step are called a few hundred times per step from Python: with their argument
        # types declared, plain integers go in without a ctypes object being made for each (a third of a call's cost).
        P, L, I, F = c_void_p, c_long, c_int, c_float
        l.llmi_gemm_tc.argtypes = [P, L, P, L, P, P, L, I, I, I, I, P, L, P, I, P, P]
        l.llmi_rmsnorm.argtypes = [I, P, P, P, P, I, I, F, P]
        l.llmi_rope_store.argtypes = [I, P, L, P, I, P, P, P, I, I, P, P, I, I, I, I, I, P]
        l.llmi_attention_prefill_tc.argtypes = [P, L, L, P, L, P, P, L, P, I, P, P, I, I, I, I, I, F, I, I, I, P, L, P, I, P, I, P, P, L, P, I, P, L, P]
        _configured = True
    return l


# ---------------------------------------------------------------------------------------------

def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = fp32(table[ids[t]]) * scale; ids int32 [T]; out fp32 [T, W]; a negative id gives zeros."""
    _need_cuda(table, ids, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous() and out.is_contiguous()
    T, W = out.shape
    _check("embed", lib().llmi_embed(c_int(_dtype_code(table)), _ptr(table), _ptr(ids), _ptr(out), c_int(T),
                                     c_int(W), c_float(scale), _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> None:
    """out[r] = weight * (x[src] * rsqrt(mean(x[src]^2) + eps)), src = rows[r] if rows is given else r."""
    _need_cuda(x, weight, out, rows)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    n, W = out.shape
    assert x.shape[1] == W and weight.numel() == W
    _check("rmsnorm", lib().llmi_rmsnorm(_dtype_code(out), x.data_ptr(), weight.data_ptr(), out.data_ptr(), _addr(rows), n, W,
                                         eps, _stream_int()))


def layernorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None,
              weight2: torch.Tensor | None = None, out2: torch.Tensor | None = None) -> None:
    """out[r] = (x[src] - mean) / sqrt(var + eps) * weight (no bias; var the mean of the squared deviations), src =
    rows[r] if rows is given else r.  With ``weight2`` and ``out2`` a second norm of the same rows leaves in the same
    pass (a layer whose two branches read the same x shares the row's mean and variance)."""
    _need_cuda(x, weight, out, rows, weight2, out2)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    n, W = out.shape
    assert x.shape[1] == W and weight.numel() == W and (weight2 is None) == (out2 is None)
    if out2 is not None:
        assert out2.shape == out.shape and out2.dtype == out.dtype and out2.is_contiguous() and weight2.dtype == torch.float32
        assert weight2.numel() == W
    _check("layernorm", lib().llmi_layernorm(c_int(_dtype_code(out)), _ptr(x), _ptr(weight), _ptr(out), _ptr(weight2), _ptr(out2),
                                             _ptr(rows), c_int(n), c_int(W), c_float(eps), _stream()))


def depth_mix(x: torch.Tensor, history: torch.Tensor, n: int, coeffs: torch.Tensor) -> None:
    """history[n] = x; then x = sum over j <= n of coeffs[j] * history[j] (j ascending, fp32).  x fp32 [T, W] contiguous;
    history fp32 [>= n + 1, T, W] contiguous; coeffs fp32 [n + 1] on the device."""
    _need_cuda(x, history, coeffs)
    assert x.dtype == history.dtype == coeffs.dtype == torch.float32 and x.is_contiguous() and history.is_contiguous()
    assert history.shape[1:] == x.shape and history.shape[0] > n and coeffs.numel() == n + 1 and coeffs.is_contiguous()
    _check("depth_mix", lib().llmi_depth_mix(_ptr(x), _ptr(history), c_long(x.numel()), c_int(n), _ptr(coeffs), _stream()))


def mix_layernorm(x: torch.Tensor, history: torch.Tensor, n: int, coeffs: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                  eps: float, weight2: torch.Tensor | None = None, out2: torch.Tensor | None = None) -> bool:
    """:func:`depth_mix` and, of the new x, :func:`layernorm` (one weight or two) in one kernel: the same x and history as
    the two leave.  False (and nothing done) where the fused form does not apply: rows that are no whole 16-byte pieces,
    widths over 4,096."""
    _need_cuda(x, history, coeffs, weight, out, weight2, out2)
    T, W = x.shape
    assert x.dtype == history.dtype == coeffs.dtype == weight.dtype == torch.float32 and x.is_contiguous() and history.is_contiguous()
    assert history.shape[1:] == x.shape and history.shape[0] > n and coeffs.numel() == n + 1 and coeffs.is_contiguous()
    assert out.shape == (T, W) and out.is_contiguous() and weight.numel() == W and (weight2 is None) == (out2 is None)
    if out2 is not None:
        assert out2.shape == out.shape and out2.dtype == out.dtype and out2.is_contiguous() and weight2.dtype == torch.float32
        assert weight2.numel() == W
    rc = lib().llmi_mix_layernorm(c_int(_dtype_code(out)), _ptr(x), _ptr(history), c_int(n), _ptr(coeffs), _ptr(weight), _ptr(out),
                                  _ptr(weight2), _ptr(out2), c_int(T), c_int(W), c_float(eps), _stream())
    if rc == -5:          # not a size of the fused form
        return False
    _check("mix_layernorm", rc)
    return True


def gate_rows(a: torch.Tensor, z: torch.Tensor) -> None:
    """a[t, :] *= logistic(z[t]) in place; z fp32, one number per row (any row stride)."""
    _need_cuda(a, z)
    T, W = a.shape
    assert a.stride(1) == 1 and z.dtype == torch.float32 and z.shape[0] == T
    _check("gate_rows", lib().llmi_gate_rows(c_int(_dtype_code(a)), _ptr(a), c_long(a.stride(0)), c_int(W), _ptr(z),
                                             c_long(z.stride(0)), c_int(T), _stream()))


ACT_SILU, ACT_GELU_TANH = 0, 1
ACTIVATIONS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH}
EXPERT_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu2": 2, "gelu": 3}      # of the routed experts' kernels (relu2: the square of relu; gelu: the exact form)
FUSED_GATE_MODES = {ACT_SILU: OUT_SWIGLU, ACT_GELU_TANH: OUT_GEGLU}     # activation -> the output mode of the products that gate in their epilogue


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, act: int = ACT_SILU) -> None:
    """out = act(gate_up[:, :F]) * gate_up[:, F:]; act: silu or the tanh form of GELU."""
    _need_cuda(gate_up, out)
    n, F = out.shape
    assert gate_up.shape == (n, 2 * F) and gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype
    _check("swiglu", lib().llmi_swiglu(c_int(_dtype_code(out)), _ptr(gate_up), _ptr(out), c_int(n), c_int(F), c_int(act), _stream()))


def linear_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
                mode: int = OUT_STORE) -> None:
    """out (mode) x·wᵀ + bias with fp32 FMA arithmetic; x [M,K], w [N,K], rows may be strided."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and x.dtype == w.dtype
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if mode == OUT_STORE:
        assert out.dtype == x.dtype
    else:
        assert out.dtype == torch.float32
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    _check("linear_simt", lib().llmi_linear_simt(
        c_int(_dtype_code(x)), _ptr(x), c_long(x.stride(0)), _ptr(w), c_long(w.stride(0)), _ptr(bias), _ptr(out),
        c_long(out.stride(0)), c_int(M), c_int(N), c_int(K), c_int(mode), _stream()))


class _TcScratch:
    """Per-device scratch of the tensor-core product: split-K partial tiles, tile tickets (zero between
    launches) and an error word that a bounded wait sets instead of hanging."""
    WORKSPACE_BYTES = 32 << 20
    N_TICKETS = 4096
    N_ATTN_TICKETS = 1 << 16

    def __init__(self, device):
        self.workspace = torch.empty(self.WORKSPACE_BYTES // 4, dtype=torch.float32, device=device)
        self.tickets = torch.zeros(self.N_TICKETS, dtype=torch.int32, device=device)
        self.attn_tickets = torch.zeros(self.N_ATTN_TICKETS, dtype=torch.int32, device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)


_tc_scratch: dict = {}


def tc_scratch(device) -> _TcScratch:
    key = torch.device(device).index or 0
    if key not in _tc_scratch:
        _tc_scratch[key] = _TcScratch(device)
    return _tc_scratch[key]


def check_device_errors(device) -> None:
    """Raise if a kernel's bounded wait gave up since the last check (synchronises the device)."""
    sc = _tc_scratch.get(torch.device(device).index or 0)
    if sc is not None:
        code = int(sc.error.item())
        if code:
            sc.error.zero_()
            raise KernelError(f"a bounded wait inside a kernel timed out (code {code}); results are invalid")


_sm_count = None


def sm_count() -> int:
    """Streaming multiprocessors of the device the kernels run on (asked once; a B200 has 148)."""
    global _sm_count
    if _sm_count is None:
        _sm_count = max(1, int(lib().llmi_sm_count()))
    return _sm_count


def gemm_tc_eligible(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
            mode: int = OUT_STORE) -> None:
    """out (mode) x·wᵀ + bias on the tcgen05 tensor cores; bf16 inputs, fp32 accumulation."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N // 2 if mode in _GATED else N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    assert out.dtype == (torch.bfloat16 if mode in (*_STORES, *_GATED) else torch.float32)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    sc = tc_scratch(x.device)
    _check("gemm_tc", lib().llmi_gemm_tc(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _addr(bias), out.data_ptr(), out.stride(0), M, N, K, mode,
        sc.workspace.data_ptr(), sc.WORKSPACE_BYTES, sc.tickets.data_ptr(), sc.N_TICKETS, sc.error.data_ptr(), _stream_int()))


class DeferredNorm:
    """A row-wise norm y = weight * x / sqrt(mean(x^2) + eps) split over the two products around it.

    The product that last updates x (a residual add) fills ``h`` = compute-type(weight * x) and ``ss`` — the sum
    of x^2 over each 16-row tile of its output, per token — and the product that reads the norm's output
    takes ``h`` as its input and multiplies its accumulators by 1/sqrt(sum(ss)/width + eps) (a reader that cannot
    do that runs the norm the plain way over ``source``, the x the filling product updated).  A norm of a
    handful of rows is all launch and latency; this way it costs no kernel.  Made by a norm part
    (``deferred``), filled by ``linear(..., then_norm=)``, consumed by passing it as ``linear``'s input.
    """
    SS_STRIDE = 64

    def __init__(self, weight: torch.Tensor, eps: float, h: torch.Tensor, ss: torch.Tensor):
        self.weight, self.eps, self.h, self.ss = weight, float(eps), h, ss
        self.source = None       # the x that the filling product updated: a reader that cannot scale normalises from it
        self.n_tiles = (h.shape[1] + 15) // 16
        assert ss.dtype == torch.float32 and ss.numel() >= self.n_tiles * self.SS_STRIDE and weight.dtype == torch.float32

    @property
    def shape(self):
        return self.h.shape

    @property
    def dtype(self):
        return self.h.dtype


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
                mode: int = OUT_STORE, then_norm: DeferredNorm | None = None, scale_from: DeferredNorm | None = None) -> None:
    """The same product for at most 64 tokens: the weight-streaming kernel (``csrc/gemm_skinny.cu``).

    ``then_norm`` (mode OUT_ADD_F32): also fill that deferred norm from the updated ``out``.
    ``scale_from``: ``x`` is that deferred norm's ``h``; apply its scale to the accumulators."""
    _need_cuda(x, w, out, bias)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N // 2 if mode in _GATED else N)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    assert out.dtype == (torch.bfloat16 if mode in (*_STORES, *_GATED) else torch.float32)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    if then_norm is not None:
        assert mode == OUT_ADD_F32 and then_norm.h.shape == (M, N) and then_norm.h.dtype == torch.bfloat16
        assert then_norm.weight.numel() == N and then_norm.h.stride(1) == 1
    if scale_from is not None:
        assert scale_from.h.data_ptr() == x.data_ptr() and scale_from.h.shape == (M, K)
    sc = tc_scratch(x.device)
    e, f = then_norm, scale_from
    if e is not None:
        e.source = out
    _check("gemm_skinny", lib().llmi_gemm_skinny(
        _ptr(x), c_long(x.stride(0)), _ptr(w), c_long(w.stride(0)), _ptr(bias), _ptr(out), c_long(out.stride(0)),
        c_int(M), c_int(N), c_int(K), c_int(mode),
        _ptr(e.weight if e else None), _ptr(e.h if e else None), c_long(e.h.stride(0) if e else 0), _ptr(e.ss if e else None),
        _ptr(f.ss if f else None), c_int(f.n_tiles if f else 0), c_float(f.eps if f else 0.0),
        _ptr(sc.error), _stream()))


SKINNY_MAX_TOKENS = 16
_FORCE_SIMT = os.environ.get("LLMI_LINEAR", "") == "simt"
_NO_SKINNY = os.environ.get("LLMI_LINEAR", "") == "tc"
_FUSE_NORM = os.environ.get("LLMI_FUSE_NORM", "1") != "0"


SKINNY_SMALL_WEIGHT = 16 << 20    # elements: up to here the weight-streaming kernel also takes 17 to 32 tokens
SKINNY_TINY_WEIGHT = 3 << 20      # and up to here 33 to 64 tokens


def skinny_applies(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the product x·wᵀ goes to the weight-streaming kernel: up to 16 tokens always; beyond, where the tcgen05
    kernel's fixed cost (cluster, TMEM, exchange of partial tiles over a cluster when there are few 128-row tiles: 4 to
    5 us) is most of its time, or where the norm that rides on the weight-streaming products would cost a kernel of
    its own.  Measured (us, weight-streaming against tcgen05), 32 tokens: 2,048 x 2,048 4.9 / 5.2, 6,144 x 2,048
    10.7 / 8.8 (plus a norm of 3 us), 2,048 x 8,192 11.3 / 11.4, but 16,384 x 2,048 21.2 / 14.8, 6,144 x 4,096
    17.2 / 13.0; 64 tokens: 576 x 1,536 5.3 / 5.5, 1,600 x 960 4.7 / 5.5, 960 x 2,560 6.9 / 6.5, but 2,048 x 2,048
    6.5 / 6.2, 2,048 x 8,192 15.2 / 12.2, 6,144 x 2,048 16.2 / 9.4, 16,384 x 2,048 32.7 / 15.4 (a decode step of the
    1.7B shape at batch 64 with the two 2,048-row products on the tcgen05 kernel: 9.61 -> 9.28 ms)."""
    n = x.shape[0]
    if _FORCE_SIMT or _NO_SKINNY or x.shape[1] % 64 or not gemm_tc_eligible(x, w):
        return False
    return bool(n <= SKINNY_MAX_TOKENS or (n <= 32 and w.numel() <= SKINNY_SMALL_WEIGHT)
                or (n <= 64 and w.numel() <= SKINNY_TINY_WEIGHT))


def norm_deferrable(n_tokens: int, width: int, dtype) -> bool:
    """Whether a norm over ``width`` of ``n_tokens`` rows can be split over the products around it."""
    return bool(_FUSE_NORM and not _FORCE_SIMT and not _NO_SKINNY and dtype == torch.bfloat16
                and n_tokens <= DeferredNorm.SS_STRIDE and width % 64 == 0)


def gemm_bf16(x, w, out, bias=None, mode: int = OUT_STORE, then_norm: DeferredNorm | None = None) -> bool:
    """The bf16 tensor-core product: the weight-streaming kernel for a handful of tokens, the tcgen05
    kernel for more.  ``x`` may be a filled :class:`DeferredNorm`; returns whether ``then_norm`` was filled."""
    pending = x if isinstance(x, DeferredNorm) else None
    xin = pending.h if pending is not None else x
    if skinny_applies(xin, w):
        gemm_skinny(xin, w, out, bias, mode, then_norm, pending)
        return then_norm is not None
    if pending is not None:
        # this reader cannot apply the scale to its accumulators: the norm is run the plain way after all, over the
        # h that the filling product left (one launch, as without the deferral)
        if pending.source is None:
            raise KernelError("a deferred norm that no product has filled")
        rmsnorm(pending.source, pending.weight, pending.h, pending.eps)
    gemm_tc(xin, w, out, bias, mode)
    return False


def linear(x, w, out, bias=None, mode: int = OUT_STORE, then_norm: DeferredNorm | None = None) -> bool:
    """The matrix product of the step: the tensor-core kernels for bf16 operands they can take (16-byte
    aligned rows), the fp32 FMA kernel for the 32-bit path and for everything else.  ``x`` may be a filled
    :class:`DeferredNorm`; returns whether ``then_norm`` was filled (False: run that norm the plain way)."""
    xin = x.h if isinstance(x, DeferredNorm) else x
    if not _FORCE_SIMT and gemm_tc_eligible(xin, w):
        return gemm_bf16(x, w, out, bias, mode, then_norm)
    if isinstance(x, DeferredNorm):      # a reader that cannot scale: the norm the plain way after all
        if x.source is None:
            raise KernelError("a deferred norm that no product has filled")
        rmsnorm(x.source, x.weight, x.h, x.eps)
    if mode in _STORE_ACTIVATIONS:       # the fp32 FMA product has no activation in its epilogue: two steps
        linear_simt(xin, w, out, bias, OUT_STORE)
        activate(out, out, _STORE_ACTIVATIONS[mode])
        return False
    linear_simt(xin, w, out, bias, mode)
    return False


def rope_store(qkv: torch.Tensor, inv_freq: torch.Tensor | None, rotary_dim: int, tok_seq, tok_pos, seq_pages,
               page_size: int, k_cache: torch.Tensor, v_cache: torch.Tensor, n_heads: int, n_kv_heads: int,
               head_dim: int, write_kv: bool = True) -> None:
    """Rotate q (in place) and k, and append k, v of each token to its sequence's cache page."""
    _need_cuda(qkv, inv_freq, tok_seq, tok_pos, seq_pages, k_cache, v_cache)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    assert seq_pages.dtype == torch.int32 and seq_pages.dim() == 2
    _check("rope_store", lib().llmi_rope_store(
        _dtype_code(qkv), qkv.data_ptr(), qkv.stride(0), _addr(inv_freq), rotary_dim, tok_seq.data_ptr(), tok_pos.data_ptr(),
        seq_pages.data_ptr(), seq_pages.stride(0), page_size, k_cache.data_ptr(), v_cache.data_ptr(), T, n_heads, n_kv_heads,
        head_dim, 1 if write_kv else 0, _stream_int()))


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, tok_seq, tok_pos, seq_pages,
                      page_size: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal attention of every token over its sequence's cache; q is [T, >= n_heads*head_dim] (row-strided)."""
    _need_cuda(q, out, k_cache, v_cache, tok_seq, tok_pos, seq_pages)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, n_heads * head_dim)
    assert q.dtype == out.dtype == k_cache.dtype
    _check("attention_generic", lib().llmi_attention_generic(
        c_int(_dtype_code(q)), _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache),
        _ptr(v_cache), _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_pages), c_int(seq_pages.stride(0)), c_int(page_size),
        c_int(T), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_int(window), _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of logits[r]; logits fp32 [R, V], out int32 [R]."""
    _need_cuda(logits, out)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    _check("argmax", lib().llmi_argmax(_ptr(logits), c_long(logits.stride(0)), c_int(R), c_int(V), _ptr(out), _stream()))


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, uniforms: torch.Tensor,
           probs_scratch: torch.Tensor, out: torch.Tensor) -> None:
    """Temperature / top-k / top-p sampling; uniforms float64 [R] in [0, 1); probs_scratch fp32 [R, V]."""
    _need_cuda(logits, uniforms, probs_scratch, out)
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert uniforms.dtype == torch.float64 and uniforms.numel() >= R
    assert probs_scratch.dtype == torch.float32 and probs_scratch.numel() >= R * V and probs_scratch.is_contiguous()
    _check("sample", lib().llmi_sample(_ptr(logits), c_long(logits.stride(0)), c_int(R), c_int(V),
                                       c_float(temperature), c_int(top_k), c_float(top_p), _ptr(uniforms),
                                       _ptr(probs_scratch), _ptr(out), _stream()))


DECODE_PAGES_PER_SPLIT = 8     # default split of the decode kernel: 512 positions


_resident_cache: dict = {}


# Which decode kernel takes grouped queries (group = query heads per kv head >= 2) of head size 64 or 128: "mma"
# (the group's heads as rows of tensor-core tiles: the work per page does not grow with the group) or "simt"
# (the CUDA-core kernel, which always takes group 1).
_DECODE_ATTENTION = os.environ.get("LLMI_DECODE_ATTENTION", "mma")


def decode_uses_mma(head_dim: int, group: int) -> bool:
    return bool(_DECODE_ATTENTION == "mma" and group >= 2
                and lib().llmi_attention_decode_mma_supported(c_int(head_dim), c_int(group)))


def decode_pages_per_split(n_seqs: int, n_kv_heads: int, max_pages: int, head_dim: int = 64, group: int = 1) -> int:
    """How many pages one work item of the decode kernel covers.

    The kernel is persistent: ``resident`` blocks share the items round-robin.  The split is chosen so
    that the last round of items is nearly full (little idle tail) while an item stays long enough
    (at least 8 pages unless the batch is tiny) that its fixed cost — first load, merge, ticket —
    is small beside its streaming time.  Large batches get no split at all.
    """
    pairs = max(1, n_seqs * n_kv_heads)
    if decode_uses_mma(head_dim, group):
        key = (head_dim, group)
        if key not in _resident_cache:
            _resident_cache[key] = max(1, int(lib().llmi_attention_decode_mma_resident(c_int(head_dim), c_int(group))))
        resident = _resident_cache[key]
        # The tensor-core kernel: the end of an item that is one of several splits costs about six pages of streaming
        # (four warps merged, the partial result written, a ticket), of a whole sequence-head two; the last split to
        # arrive merges two heads and NZ splits per round trip to L2 (about 1.5 pages of head size 64 each).
        # Measured at 4,096 positions: 8 kv heads of size 64, batch 1: 8.7 us at 4 pages a split, 10.6 at 2, 13.1 at
        # 16; batch 64: 84 us without splits, 91 at 16 pages, 119 at 8.
        nz = 16 if head_dim <= 64 else 8
        best, best_cost = max_pages, float("inf")
        for splits in range(1, max(1, max_pages // 4) + 1):
            pps = -(-max_pages // splits)
            n_parts = -(-max_pages // pps)
            rounds = -(-pairs * n_parts // resident)
            cost = rounds * (pps + (2 if n_parts == 1 else 6))
            if n_parts > 1:
                cost += -(-group // 2) * -(-n_parts // nz) * 1.5 * 64 / head_dim
            if cost < best_cost - 1e-9:
                best, best_cost = pps, cost
        return best
    # The CUDA-core kernel has two variants (csrc/attention_decode.cu): with few sequence-heads the one with a producer
    # thread for the key tiles and one for the value tiles, two blocks per SM, whose items may be long.
    key = (head_dim, group, n_seqs, n_kv_heads)
    if key not in _resident_cache:
        two = ctypes.c_int(0)
        resident = int(lib().llmi_attention_decode_plan(c_int(head_dim), c_int(group), c_int(n_seqs), c_int(n_kv_heads), ctypes.byref(two)))
        _resident_cache[key] = (max(1, resident), bool(two.value))
    resident, two_producers = _resident_cache[key]
    best, best_score = max_pages, -1.0
    for splits in range(1, max(1, max_pages // (2 if two_producers else 4)) + 1):
        pps = -(-max_pages // splits)
        n_parts = -(-max_pages // pps)
        items = pairs * n_parts
        rounds = -(-items // resident)
        fill = items / (rounds * resident)                 # how full the rounds are
        # An item costs about two pages of streaming on top; with two producers, where items are read twice as fast,
        # one of several splits about four (partial result, fence, ticket, the last one's merge).  The latter fitted
        # to measurements (32 kv heads of 64; best split measured = chosen): 4,096 positions at batch 1 / 2 / 4 / 8:
        # 8 / 16 / 32 pages / none; 8,192 positions: 16 / 32 / 64 / none; 1,024 positions: 2 / 4 / 8 / none.
        score = fill * pps / (pps + (4.0 if (two_producers and n_parts > 1) else 2.0))
        if score > best_score + 1e-9:
            best, best_score = pps, score
    return best


_PLAN_BY_LIVE = os.environ.get("LLMI_DECODE_PLAN", "live") != "padded"
_plan_cache: dict = {}


def decode_plan(ctx, n_seqs: int, n_pages: int, page_size: int, n_kv_heads: int, head_dim: int, group: int):
    """(pages per item, live sequences) for the decode kernel of a step whose page tables are [n_seqs, n_pages].

    A recorded step is padded to a power of two of sequences.  The kernel skips the padding, but a split chosen for
    16 sequences is a poor one for 9 or 12: so the split (and the kernel's variant) follow the step's LIVE sequences
    (:func:`decode_plan_token` tells recorded steps with different answers apart).  Measured, a decode step of 32
    heads of 64 at 4,096 positions, planned by the padded and by the live number: batch 3 1.334 -> 1.291 ms, 5
    1.754 -> 1.597, 9 2.145 -> 2.025, 12 2.594 -> 2.403, 24 4.264 -> 4.165; 14 and 40 unchanged.  The page tables'
    padded width stays the measure of length: following the live pages too changed the split every few hundred
    tokens (a new recording each time) for no gain at batch 1 to 3.  ``LLMI_DECODE_PLAN=padded`` plans by the
    padded number."""
    n_live = n_seqs
    if _PLAN_BY_LIVE:
        n_live = min(n_seqs, max(1, int(getattr(ctx, "n_real_seqs", 0) or n_seqs)))
    key = (n_live, n_pages, n_kv_heads, head_dim, group)
    plan = _plan_cache.get(key)
    if plan is None:
        pps = decode_pages_per_split(n_live, n_kv_heads, n_pages, head_dim, group)
        cluster = decode_cluster(n_live, n_kv_heads, n_pages, head_dim, group) if pps < n_pages else 0
        if cluster:
            pps = -(-n_pages // cluster)
        plan = _plan_cache[key] = (pps, cluster)
    return plan[0], n_live, plan[1]


_CLUSTER = os.environ.get("LLMI_DECODE_CLUSTER", "1") != "0"
_CLUSTER_MAX_PAGES = int(os.environ.get("LLMI_DECODE_CLUSTER_PAGES", "4"))
_clusters_resident: dict = {}


def decode_cluster(n_live: int, n_kv_heads: int, n_pages: int, head_dim: int, group: int) -> int:
    """The size of the clusters (8, 4 or 2 blocks, one cluster per sequence-head) in which the decode kernel runs a
    step of few sequence-heads and short sequences, or 0 for its persistent form: the largest size whose clusters are
    all resident at once and give a block two to four pages (``LLMI_DECODE_CLUSTER_PAGES``).  Ungrouped queries on the
    CUDA-core kernel only.  With so few pages a block the kernel is as long as the chain behind its last page —
    partial result to memory, fence, ticket, the last block's loads of all partial results — and the clusters replace
    that chain by stores into the first block's shared memory.  A decode step of 32 heads of 64 (24 layers, 2,048
    wide), persistent form -> clusters: batch 1 at 512 / 1,024 / 2,048 positions 0.985 -> 0.933 / 0.999 -> 0.964 /
    1.020 -> 0.995 ms; batch 2 at 512 / 1,024: 0.968 -> 0.941 / 0.997 -> 0.980; batch 4 at 512: 0.994 -> 0.984.  With
    more pages a block it loses (one producer thread a block, few blocks: batch 1 at 4,096 positions, 8 pages a
    block: 1.060 -> 1.084 ms; batch 4: 1.402 -> 1.547), so there the persistent form with its shorter items stays.
    ``LLMI_DECODE_CLUSTER=0`` switches the clusters off."""
    if not _CLUSTER or group != 1 or decode_uses_mma(head_dim, group):
        return 0
    for size in (8, 4, 2):
        if n_pages < 2 * size or -(-n_pages // size) > _CLUSTER_MAX_PAGES:
            continue
        key = (head_dim, size)
        if key not in _clusters_resident:
            _clusters_resident[key] = int(lib().llmi_attention_decode_clusters_resident(c_int(head_dim), c_int(group), c_int(size)))
        if n_live * n_kv_heads <= _clusters_resident[key]:
            return size
    return 0


def decode_plan_token(ctx, n_seqs: int, n_pages: int, page_size: int, n_kv_heads: int, head_dim: int, group: int):
    """What tells two recorded decode steps of the same padded shape apart: the split and the kernel's variant."""
    pps, n_live, cluster = decode_plan(ctx, n_seqs, n_pages, page_size, n_kv_heads, head_dim, group)
    if decode_uses_mma(head_dim, group):
        return (pps,)
    key = (head_dim, group, n_live, n_kv_heads)
    if key not in _resident_cache:
        decode_pages_per_split(n_live, n_kv_heads, n_pages, head_dim, group)
    return (pps, _resident_cache[key][1], cluster)


def attention_decode_supported(head_dim: int, group: int) -> bool:
    return decode_uses_mma(head_dim, group) or bool(lib().llmi_attention_decode_supported(c_int(head_dim), c_int(group)))


def attention_decode_mma(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start,
                         n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, partials: torch.Tensor,
                         pages_per_split: int, rope=None) -> None:
    """:func:`attention_decode` (``rope`` None) or :func:`attention_decode_fused` (``rope = (inv_freq, rotary_dim,
    write_kv)``, ``q`` the un-rotated [q | k | v] rows) by the tensor-core kernel for grouped queries."""
    _need_cuda(q, out, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start, partials)
    S, P = seq_pages.shape
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.shape[-2] == 64 and partials.dtype == torch.float32
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    inv_freq, rotary_dim, write_kv = rope if rope is not None else (None, 0, False)
    assert rotary_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2)
    sc = tc_scratch(q.device)
    _check("attention_decode_mma", lib().llmi_attention_decode_mma(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_long(k_cache.shape[0]), _ptr(seq_pages), c_int(seq_pages.stride(0)), _ptr(seq_kv_len), _ptr(seq_q_start), c_int(S),
        c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_int(window), c_int(P), c_int(pages_per_split),
        c_int(0 if rope is None else 1), _ptr(inv_freq) if rotary_dim else None, c_int(rotary_dim),
        c_int(1 if write_kv else 0), _ptr(partials), c_long(partials.numel()), _ptr(sc.attn_tickets),
        c_int(sc.N_ATTN_TICKETS), _ptr(sc.error), _stream()))


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start,
                     n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, partials: torch.Tensor,
                     pages_per_split: int = DECODE_PAGES_PER_SPLIT, n_live: int = 0, cluster: int = 0) -> None:
    """One token per sequence over its cache pages (bf16, page size 64), split over positions.

    ``partials``: fp32 scratch of at least ``attention_decode_workspace(...)`` floats.  ``n_live``: how many of
    the sequences are not padding, if the caller knows (it decides which variant of the kernel runs, nothing else).
    ``cluster`` (2, 4, 8; ungrouped queries): the form of the kernel with one cluster of that many blocks per
    sequence-head, whose splits meet in shared memory; ``pages_per_split`` x ``cluster`` must cover the page tables.
    """
    _need_cuda(q, out, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start, partials)
    S, P = seq_pages.shape
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and k_cache.shape[-2] == 64 and partials.dtype == torch.float32
    sc = tc_scratch(q.device)
    _check("attention_decode", lib().llmi_attention_decode(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(seq_pages),
        c_int(seq_pages.stride(0)), _ptr(seq_kv_len), _ptr(seq_q_start), c_int(S), c_int(n_heads), c_int(n_kv_heads),
        c_int(head_dim), c_float(scale), c_int(window), c_int(P), c_int(pages_per_split), _ptr(partials),
        c_long(partials.numel()), _ptr(sc.attn_tickets), c_int(sc.N_ATTN_TICKETS), _ptr(sc.error), c_int(n_live),
        c_int(cluster), _stream()))


def attention_decode_workspace(n_seqs: int, n_heads: int, head_dim: int, max_pages: int,
                               pages_per_split: int = DECODE_PAGES_PER_SPLIT) -> int:
    return int(lib().llmi_attention_decode_workspace(c_int(n_seqs), c_int(n_heads), c_int(head_dim), c_int(max_pages),
                                                     c_int(pages_per_split)))


def attention_prefill_supported(head_dim: int) -> bool:
    return bool(lib().llmi_attention_prefill_supported(c_int(head_dim)))


def attention_prefill_tc_supported(head_dim: int) -> bool:
    return bool(lib().llmi_attention_prefill_tc_supported(c_int(head_dim)))


def attention_prefill(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, seq_pages, seq_q_start, seq_kv_len,
                      n_blocks: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal attention of the prompts of a step over their cache pages (bf16, head size 64 or 128, page 64).

    ``seq_q_start`` [n_seqs + 1] are the sequences' offsets into the step's tokens, ``seq_kv_len`` their
    lengths after the step, ``n_blocks`` the sum over sequences of ceil(tokens / 128).
    """
    _need_cuda(q, out, k_cache, v_cache, seq_pages, seq_q_start, seq_kv_len)
    S = seq_pages.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert k_cache.shape[-2] == 64 and k_cache.is_contiguous() and v_cache.is_contiguous()
    sc = tc_scratch(q.device)
    _check("attention_prefill", lib().llmi_attention_prefill(
        _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache),
        c_long(k_cache.shape[0]), _ptr(seq_pages), c_int(seq_pages.stride(0)), _ptr(seq_q_start), _ptr(seq_kv_len),
        c_int(S), c_int(n_blocks), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_float(scale), c_int(window),
        _ptr(sc.error), _stream()))


PREFILL_SPLIT_PAGES = 16      # key pages per job when the prompt attention cuts its long query blocks


def prefill_split_jobs(q_lens, kv_lens, window: int, split_pages: int, pool: int = 0) -> int:
    """How many jobs the prompt attention has along its first grid dimension when every block of 128 queries
    is cut into parts of ``split_pages`` key pages (the kernel's own rule, counted on the host).  ``pool``: pages of
    pooled rows (one per ``pool`` positions that lie before the window) come ahead of a block's own pages."""
    jobs = 0
    for q_len, kv_len in zip(q_lens, kv_lens):
        pos0 = kv_len - q_len
        for mb in range((q_len + 127) // 128):
            first_q = pos0 + mb * 128
            last_q = first_q + min(128, q_len - mb * 128) - 1
            lo_key = first_q - window + 1 if (window > 0 and first_q - window + 1 > 0) else 0
            n_pg = last_q // 64 - lo_key // 64 + 1
            if pool > 0 and last_q - window + 1 > 0:
                n_pg += ((last_q - window + 1) // pool + 63) // 64
            jobs += (n_pg + split_pages - 1) // split_pages
    return jobs


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, seq_pages, seq_q_start, seq_kv_len,
                         n_blocks: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                         split=None, pooled=None, gate=None) -> None:
    """The same prompt attention on the tcgen05 tensor cores (head size 64 or 128); arguments as ``attention_prefill``.
    ``pooled = (pool, k_pool, v_pool, pool_pages)``: beside its window a query sees one pooled row per block of ``pool``
    positions that lies wholly before the window (row b of the sequence's pooled pages is block b; caches shaped as the
    token caches).  ``gate``: fp32 [tokens, >= n_heads]; head h's output is multiplied by logistic(gate[t, h]).
    ``split = (n_jobs, split_pages, workspace)``: cut the key range of every query block into jobs of
    ``split_pages`` pages (``n_jobs`` from :func:`prefill_split_jobs`, ``workspace`` fp32 of
    n_jobs * n_heads * (head_dim + 2) * 128 floats)."""
    _need_cuda(q, out, k_cache, v_cache, seq_pages, seq_q_start, seq_kv_len)
    S = seq_pages.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert k_cache.shape[-2] == 64 and k_cache.is_contiguous() and v_cache.is_contiguous()
    sc = tc_scratch(q.device)
    n_jobs, split_pages, ws = split if split is not None else (n_blocks, 0, None)
    if ws is not None:
        assert ws.dtype == torch.float32 and ws.is_cuda
    pool, k_pool, v_pool, pool_pages = pooled if pooled is not None else (0, None, None, None)
    if pool:
        _need_cuda(k_pool, v_pool, pool_pages)
        assert window > 0 and k_pool.dtype == v_pool.dtype == torch.bfloat16 and pool_pages.dtype == torch.int32
        assert k_pool.is_contiguous() and v_pool.is_contiguous() and k_pool.shape[1:] == k_cache.shape[1:] == v_pool.shape[1:]
        assert pool_pages.shape[0] == S and pool_pages.stride(1) == 1
    if gate is not None:
        _need_cuda(gate)
        assert gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == q.shape[0] and gate.shape[1] >= n_heads
    _check("attention_prefill_tc", lib().llmi_attention_prefill_tc(
        q.data_ptr(), q.stride(0), q.shape[0], out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
        k_cache.shape[0], seq_pages.data_ptr(), seq_pages.stride(0), seq_q_start.data_ptr(), seq_kv_len.data_ptr(), S,
        n_blocks, n_heads, n_kv_heads, head_dim, scale, window, n_jobs, split_pages, _addr(ws),
        ws.numel() if ws is not None else 0, sc.attn_tickets.data_ptr(), sc.N_ATTN_TICKETS, sc.error.data_ptr(), pool,
        _addr(k_pool), _addr(v_pool), k_pool.shape[0] if pool else 0, _addr(pool_pages), pool_pages.stride(0) if pool else 0,
        _addr(gate), gate.stride(0) if gate is not None else 0, _stream_int()))


# Which prompt-attention kernel runs: "tc" (tcgen05: about 43 us for a 2,048-token prompt of 32 heads of 64) or
# "mma" (mma.sync: 95 us).
_PREFILL_ATTENTION = os.environ.get("LLMI_PREFILL_ATTENTION", "tc")     # "mma": the mma.sync kernel for every head size
_FORCE_GENERIC_ATTENTION = os.environ.get("LLMI_ATTENTION", "") == "generic"
_PREFILL_SPLIT = os.environ.get("LLMI_PREFILL_SPLIT", "1") != "0"


def attention_decode_fused(qkv: torch.Tensor, out: torch.Tensor, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start,
                           n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, partials: torch.Tensor,
                           pages_per_split: int, inv_freq, rotary_dim: int, write_kv: bool, n_live: int = 0,
                           cluster: int = 0) -> None:
    """:func:`attention_decode` with the step's position encoding done by the same kernel: ``qkv`` holds the
    un-rotated [q | k | v] row of each sequence's token; the new k (rotated) and v are appended to the cache."""
    _need_cuda(qkv, out, k_cache, v_cache, seq_pages, seq_kv_len, seq_q_start, partials)
    S, P = seq_pages.shape
    assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
    assert qkv.stride(1) == 1 and out.stride(1) == 1 and k_cache.shape[-2] == 64 and partials.dtype == torch.float32
    assert rotary_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2)
    sc = tc_scratch(qkv.device)
    _check("attention_decode_fused", lib().llmi_attention_decode_fused(
        _ptr(qkv), c_long(qkv.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(seq_pages),
        c_int(seq_pages.stride(0)), _ptr(seq_kv_len), _ptr(seq_q_start), c_int(S), c_int(n_heads), c_int(n_kv_heads),
        c_int(head_dim), c_float(scale), c_int(window), c_int(P), c_int(pages_per_split),
        _ptr(inv_freq) if rotary_dim else None, c_int(rotary_dim), c_int(1 if write_kv else 0), _ptr(partials),
        c_long(partials.numel()), _ptr(sc.attn_tickets), c_int(sc.N_ATTN_TICKETS), _ptr(sc.error), c_int(n_live),
        c_int(cluster), _stream()))


_FUSE_ROPE = os.environ.get("LLMI_FUSE_ROPE", "1") != "0"


def _decode_kernel_applies(qkv, ctx, seq_pages, page_size, n_heads, n_kv_heads, head_dim, rt) -> bool:
    return bool(ctx.decode and qkv.dtype == torch.bfloat16 and page_size == 64 and rt is not None
                and not _FORCE_GENERIC_ATTENTION and seq_pages.shape[0] * n_kv_heads <= _TcScratch.N_ATTN_TICKETS
                and attention_decode_supported(head_dim, n_heads // n_kv_heads))


def attention_fuses_rotation(qkv, ctx, seq_pages, page_size, n_heads, n_kv_heads, head_dim, rotary_dim, rt) -> bool:
    """Whether :func:`attention` can do this step's rotation and cache append itself (``rope=``): a decode
    step that goes to the split kernel, rotating the whole head or nothing."""
    return bool(_FUSE_ROPE and rotary_dim in (0, head_dim)
                and _decode_kernel_applies(qkv, ctx, seq_pages, page_size, n_heads, n_kv_heads, head_dim, rt))


def attention(qkv: torch.Tensor, out: torch.Tensor, k_cache, v_cache, ctx, seq_pages, page_size: int, n_heads: int,
              n_kv_heads: int, head_dim: int, scale: float, window: int = 0, rt=None, rope=None) -> None:
    """Attention of a step's tokens over the cache; q is the first n_heads*head_dim columns of ``qkv``.

    In bf16, a decode step goes to the split kernel and a prompt step to the flash kernel when they
    have the head size; everything else (the 32-bit path, other head sizes) goes to the generic kernel.
    ``rope=(inv_freq, rotary_dim, write_kv)``: q, k are not rotated yet and k, v not appended — the kernel
    does it (only where :func:`attention_fuses_rotation` says so).
    """
    if _decode_kernel_applies(qkv, ctx, seq_pages, page_size, n_heads, n_kv_heads, head_dim, rt):
        S, P = seq_pages.shape
        pps, n_live, cluster = decode_plan(ctx, S, P, page_size, n_kv_heads, head_dim, n_heads // n_kv_heads)
        partials = rt.scratch("attn_partials", (attention_decode_workspace(S, n_heads, head_dim, P, pps),), torch.float32)
        if decode_uses_mma(head_dim, n_heads // n_kv_heads):
            attention_decode_mma(qkv, out, k_cache, v_cache, seq_pages, ctx.seq_kv_len, ctx.seq_q_start, n_heads,
                                 n_kv_heads, head_dim, scale, window, partials, pps, rope)
        elif rope is not None:
            attention_decode_fused(qkv, out, k_cache, v_cache, seq_pages, ctx.seq_kv_len, ctx.seq_q_start, n_heads,
                                   n_kv_heads, head_dim, scale, window, partials, pps, rope[0], rope[1], rope[2], n_live,
                                   cluster)
        else:
            attention_decode(qkv, out, k_cache, v_cache, seq_pages, ctx.seq_kv_len, ctx.seq_q_start, n_heads, n_kv_heads,
                             head_dim, scale, window, partials, pps, n_live, cluster)
        return
    if rope is not None:
        raise RuntimeError("attention: rotation can only be fused into the decode kernel (ask attention_fuses_rotation)")
    if (not ctx.decode and qkv.dtype == torch.bfloat16 and page_size == 64 and not _FORCE_GENERIC_ATTENTION
            and attention_prefill_supported(head_dim)):
        if (_PREFILL_ATTENTION == "tc" and attention_prefill_tc_supported(head_dim) and qkv.stride(0) % 8 == 0
                and out.stride(0) % 8 == 0):
            # A step with fewer (query block, head) jobs than the device has SMs leaves SMs idle and is as long as its
            # longest job: then the key ranges are cut (see the kernel's head).  Measured: 2,048 tokens x 8 heads 28.0 ->
            # 22.2 us, x 4 heads 27.5 -> 21.0 us; with 256 jobs and more the cut gains nothing or costs (4,096 x 8:
            # 49.3 -> 50.5 us; 2,048 x 32: 42.1 -> 49.6 us).
            split = None
            q_lens, kv_lens = getattr(ctx, "host_q_lens", None), getattr(ctx, "host_kv_lens", None)
            if _PREFILL_SPLIT and rt is not None and q_lens is not None and ctx.n_q_blocks * n_heads < sm_count():
                jobs = prefill_split_jobs(q_lens, kv_lens, window, PREFILL_SPLIT_PAGES)
                if jobs > ctx.n_q_blocks:
                    ws = rt.scratch("attn_prefill_partials", (jobs * n_heads * (head_dim + 2) * 128,), torch.float32)
                    split = (jobs, PREFILL_SPLIT_PAGES, ws)
            attention_prefill_tc(qkv, out, k_cache, v_cache, seq_pages, ctx.seq_q_start, ctx.seq_kv_len, ctx.n_q_blocks,
                                 n_heads, n_kv_heads, head_dim, scale, window, split)
            return
        attention_prefill(qkv, out, k_cache, v_cache, seq_pages, ctx.seq_q_start, ctx.seq_kv_len, ctx.n_q_blocks,
                          n_heads, n_kv_heads, head_dim, scale, window)
        return
    attention_generic(qkv, out, k_cache, v_cache, ctx.tok_seq, ctx.tok_pos, seq_pages, page_size, n_heads,
                      n_kv_heads, head_dim, scale, window)


# ---------------------------------------------------------------------------------------------
# Attention in its general form (csrc/qkv_prepare.cu, csrc/attention_flex.cu)

def qkv_prepare(proj: torch.Tensor, n_q_heads: int, n_k_heads: int, dk: int, n_v_heads: int, dv: int, q_norm_w, k_norm_w,
                eps: float, inv_freq, rot_dims: int, ctx, seq_pages, page_size: int, k_cache, v_cache, q_out: torch.Tensor,
                has_kv: bool = True, write_kv: bool = True, pairing: int = 0, amplitude: float = 1.0,
                v_from_k: bool = False) -> None:
    """From the fp32 rows [q | k | v] of a step (k, v absent without ``has_kv``): optional RMS norms over the whole q
    part and the whole k part (weights ``q_norm_w``, ``k_norm_w``), rotation of the first ``rot_dims`` entries of every
    q and k head (``pairing`` 0: entries (i, i + rot_dims/2); 1: neighbours (2i, 2i + 1); cos and sin times
    ``amplitude``), q into ``q_out`` (compute type), k and v into their cache pages.  ``v_from_k``: the rows hold no v
    part; the values are the key rows before the rotation."""
    _need_cuda(proj, q_norm_w, k_norm_w, inv_freq, seq_pages, k_cache, v_cache, q_out)
    T = proj.shape[0]
    n_in = n_q_heads * dk + ((n_k_heads * dk + (0 if v_from_k else n_v_heads * dv)) if has_kv else 0)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and proj.shape[1] >= n_in
    assert q_out.shape == (T, n_q_heads * dk) and q_out.stride(1) == 1 and seq_pages.dtype == torch.int32
    for wt, n in ((q_norm_w, n_q_heads * dk), (k_norm_w, n_k_heads * dk)):
        assert wt is None or (wt.dtype == torch.float32 and wt.numel() == n and wt.is_contiguous())
    if has_kv:
        assert k_cache.dtype == v_cache.dtype == q_out.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
        assert k_cache.shape[-3:] == (n_k_heads, page_size, dk) and v_cache.shape[-3:] == (n_v_heads, page_size, dv)
    if rot_dims:
        assert inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() >= rot_dims // 2
    _check("qkv_prepare", lib().llmi_qkv_prepare(
        c_int(_dtype_code(q_out)), _ptr(proj), c_long(proj.stride(0)), c_int(n_q_heads), c_int(n_k_heads), c_int(dk),
        c_int(n_v_heads), c_int(dv), _ptr(q_norm_w), _ptr(k_norm_w), c_float(eps), _ptr(inv_freq), c_int(rot_dims),
        c_int(pairing), c_float(amplitude), c_int(1 if v_from_k else 0),
        _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(seq_pages), c_int(seq_pages.stride(0)), _ptr(seq_pages),
        c_int(seq_pages.stride(0)), c_int(page_size), _ptr(k_cache if has_kv else None), _ptr(v_cache if has_kv else None),
        _ptr(q_out), c_long(q_out.stride(0)), c_int(T), c_int(1 if has_kv else 0), c_int(1 if write_kv else 0), _stream()))


def attention_flex(q: torch.Tensor, out: torch.Tensor, k_cache, v_cache, ctx, seq_pages, page_size: int, n_heads: int,
                   n_kv_heads: int, maps: int, dk: int, dv: int, scale: float, head_scale=None, window: int = 0,
                   chunk: int = 0, pooled=None, gate=None, softcap: float = 0.0) -> None:
    """Causal attention of every token over its sequence's cache with ``maps`` score maps per head (query row
    [head][map][dk], key heads [kv head][map], one set of values [kv head][dv]); out [T, heads*maps*dv] in q's type or
    fp32.  ``head_scale`` fp32 [heads] multiplies the scores of a head; ``window`` and ``chunk`` limit the visible keys
    (a query at p sees max(p - window + 1, p // chunk * chunk) .. p).  ``pooled`` = (pool, k_pool, v_pool, pool_pages):
    beside its window a query sees row b of the pooled pages for every block b of ``pool`` positions that lies wholly
    before the window (b * pool + pool - 1 <= p - window), in the same softmax.  ``gate`` fp32 [T, >= heads] (row-strided):
    head h's output is multiplied by logistic(gate[t, h]); a gate of exactly heads*dv columns (one map) has a number per
    output entry instead.  ``softcap`` > 0: a score s becomes softcap * tanh(s / softcap) before the softmax."""
    gate_per = _gate_per(gate, n_heads, maps, dv)
    _need_cuda(q, out, k_cache, v_cache, seq_pages, head_scale, gate)
    T = q.shape[0]
    pool, k_pool, v_pool, pool_pages = pooled if pooled is not None else (0, None, None, None)
    if pool:
        _need_cuda(k_pool, v_pool, pool_pages)
        assert window > 0 and k_pool.dtype == v_pool.dtype == q.dtype and pool_pages.dtype == torch.int32
        assert k_pool.shape[-3:] == (n_kv_heads * maps, page_size, dk) and v_pool.shape[-3:] == (n_kv_heads, page_size, dv)
        assert k_pool.is_contiguous() and v_pool.is_contiguous() and pool_pages.shape[0] == seq_pages.shape[0]
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == T and gate.shape[1] >= n_heads)
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, n_heads * maps * dv) and q.shape[1] >= n_heads * maps * dk
    assert q.dtype == k_cache.dtype == v_cache.dtype and out.dtype in (q.dtype, torch.float32)
    assert k_cache.shape[-3:] == (n_kv_heads * maps, page_size, dk) and v_cache.shape[-3:] == (n_kv_heads, page_size, dv)
    assert head_scale is None or (head_scale.dtype == torch.float32 and head_scale.numel() == n_heads)
    _check("attention_flex", lib().llmi_attention_flex(
        c_int(_dtype_code(q)), _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)),
        c_int(1 if out.dtype == torch.float32 else 0), _ptr(k_cache), _ptr(v_cache), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos),
        _ptr(seq_pages), c_int(seq_pages.stride(0)), c_int(page_size), c_int(T), c_int(n_heads), c_int(n_kv_heads), c_int(maps),
        c_int(dk), c_int(dv), c_float(scale), _ptr(head_scale), c_int(window), c_int(chunk), c_int(pool), _ptr(k_pool), _ptr(v_pool),
        _ptr(pool_pages), c_int(pool_pages.stride(0) if pool else 0), _ptr(gate), c_long(gate.stride(0) if gate is not None else 0),
        c_int(gate_per), c_float(softcap), _stream()))


def _gate_per(gate, n_heads: int, maps: int, dv: int) -> int:
    """How an output gate is laid out: 1 — a number per (token, head); dv — a number per output entry (a gate of
    exactly heads*dv columns, one map, where that is not also the head count)."""
    if gate is None or maps != 1 or dv == 1 or gate.shape[1] != n_heads * dv:
        return 1
    return dv


def pool_rows(k_cache, v_cache, seq_pages, k_pool, v_pool, pool_pages, page_size: int, pool: int, ctx) -> None:
    """For every token of the step whose position ends a block of ``pool`` positions: the mean of the block's key rows
    and of its value rows, as the cache holds them (added in position order in fp32), into row pos // pool of the pooled
    pages (``k_pool``, ``v_pool`` with the page table ``pool_pages``)."""
    _need_cuda(k_cache, v_cache, seq_pages, k_pool, v_pool, pool_pages)
    assert k_cache.dtype == v_cache.dtype == k_pool.dtype == v_pool.dtype and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and k_pool.shape[-3:] == k_cache.shape[-3:]
    assert v_pool.shape[-3:] == v_cache.shape[-3:] and k_cache.shape[-2] == page_size and pool >= 1
    assert seq_pages.dtype == pool_pages.dtype == torch.int32 and seq_pages.shape[0] == pool_pages.shape[0]
    _check("pool_rows", lib().llmi_pool_rows(
        c_int(_dtype_code(k_cache)), _ptr(k_cache), _ptr(v_cache), _ptr(seq_pages), c_int(seq_pages.stride(0)), _ptr(k_pool),
        _ptr(v_pool), _ptr(pool_pages), c_int(pool_pages.stride(0)), c_int(page_size), c_int(k_cache.shape[-3]),
        c_int(k_cache.shape[-1]), c_int(v_cache.shape[-3]), c_int(v_cache.shape[-1]), c_int(pool), _ptr(ctx.tok_seq),
        _ptr(ctx.tok_pos), c_int(ctx.tok_seq.shape[0]), _stream()))


def attention_maps(q, out, k_cache, v_cache, ctx, seq_pages, page_size: int, n_heads: int, n_kv_heads: int, maps: int,
                   dk: int, dv: int, scale: float, head_scale=None, window: int = 0, chunk: int = 0, rt=None, pooled=None,
                   gate=None, softcap: float = 0.0) -> None:
    """The attention of a step in its general form (arguments as :func:`attention_flex`): bf16 sizes that the
    tensor-core kernel takes go there — prompts as blocks of 128 query rows, steps of single tokens cut over the
    positions (``rt`` lends the workspace of the cuts) —, everything else, and the 32-bit path, to the generic kernel."""
    gate_per = _gate_per(gate, n_heads, maps, dv)
    if (not ctx.decode and maps == 1 and chunk == 0 and head_scale is None and dk == dv and softcap == 0.0 and gate_per == 1 and page_size == 64 and scale > 0
            and q.dtype == out.dtype == k_cache.dtype == torch.bfloat16 and rt is not None and _MAPS_ATTENTION == "mma"
            and _PREFILL_ATTENTION == "tc" and not _FORCE_GENERIC_ATTENTION and attention_prefill_tc_supported(dk)
            and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
            and (pooled is None or not pooled[0] or window > 0)):
        # one map, equal head sizes, no mask of chunks: the prompt kernel of the tcgen05 tensor cores (its window, the
        # pooled rows ahead of it, the gate per head); key ranges are cut when the step has fewer jobs than the device SMs
        pool = pooled[0] if pooled is not None else 0
        split = None
        q_lens, kv_lens = getattr(ctx, "host_q_lens", None), getattr(ctx, "host_kv_lens", None)
        n_q_blocks = getattr(ctx, "n_q_blocks", None)
        if not n_q_blocks:      # exact where the lengths are known (a cut key range counts its jobs from them), else an upper bound
            n_q_blocks = sum((n + 127) // 128 for n in q_lens) if q_lens is not None else q.shape[0] // 128 + seq_pages.shape[0]
        if _PREFILL_SPLIT and q_lens is not None and n_q_blocks * n_heads < sm_count():
            jobs = prefill_split_jobs(q_lens, kv_lens, window, PREFILL_SPLIT_PAGES, pool)
            if jobs > n_q_blocks:
                ws = rt.scratch("attn_prefill_partials", (jobs * n_heads * (dk + 2) * 128,), torch.float32)
                split = (jobs, PREFILL_SPLIT_PAGES, ws)
        attention_prefill_tc(q, out, k_cache, v_cache, seq_pages, ctx.seq_q_start, ctx.seq_kv_len, n_q_blocks, n_heads,
                             n_kv_heads, dk, scale, window, split, pooled if pool else None, gate)
        return
    if (q.dtype == torch.bfloat16 and rt is not None and _MAPS_ATTENTION == "mma" and not _FORCE_GENERIC_ATTENTION
            and lib().llmi_attention_maps_mma_supported(c_int(dk), c_int(dv), c_int(n_heads // n_kv_heads), c_int(page_size))
            and q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0 and out.stride(0) % 2 == 0 and out.data_ptr() % 8 == 0):
        _need_cuda(q, out, k_cache, v_cache, seq_pages, head_scale, gate)
        T = q.shape[0]
        S, P = seq_pages.shape
        pool, k_pool, v_pool, pool_pages = pooled if pooled is not None else (0, None, None, None)
        if pool:
            _need_cuda(k_pool, v_pool, pool_pages)
            assert window > 0 and k_pool.dtype == v_pool.dtype == torch.bfloat16 and pool_pages.dtype == torch.int32
            assert k_pool.shape[-3:] == (n_kv_heads * maps, page_size, dk) and v_pool.shape[-3:] == (n_kv_heads, page_size, dv)
            assert k_pool.is_contiguous() and v_pool.is_contiguous() and pool_pages.shape[0] == S
        assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == T and gate.shape[1] >= n_heads)
        assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, n_heads * maps * dv) and k_cache.is_contiguous()
        assert v_cache.is_contiguous() and k_cache.shape[-3:] == (n_kv_heads * maps, page_size, dk)
        assert v_cache.shape[-3:] == (n_kv_heads, page_size, dv) and out.dtype in (torch.bfloat16, torch.float32)
        prompt = not ctx.decode
        splits, pps, ws, n_ws = 1, max(P, 1), None, 0
        if not prompt:
            splits, pps = maps_attention_plan(S, P, n_kv_heads * maps, window, chunk, page_size, pool)
            n_ws = int(lib().llmi_attention_maps_mma_workspace(c_int(T), c_int(n_heads), c_int(maps), c_int(dv), c_int(splits)))
            ws = rt.scratch("attn_maps_partials", (n_ws,), torch.float32)
        _check("attention_maps_mma", lib().llmi_attention_maps_mma(
            _ptr(q), c_long(q.stride(0)), _ptr(out), c_long(out.stride(0)), c_int(1 if out.dtype == torch.float32 else 0),
            _ptr(k_cache), _ptr(v_cache), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(seq_pages), c_int(seq_pages.stride(0)),
            _ptr(ctx.seq_q_start), _ptr(ctx.seq_kv_len), c_int(T), c_int(S), c_int(n_heads), c_int(n_kv_heads), c_int(maps), c_int(dk),
            c_int(dv), c_float(scale), _ptr(head_scale), c_int(window), c_int(chunk), c_int(1 if prompt else 0),
            c_int(T // 128 + S), c_int(splits), c_int(pps), _ptr(ws), c_long(n_ws), c_int(pool), _ptr(k_pool), _ptr(v_pool),
            _ptr(pool_pages), c_int(pool_pages.stride(0) if pool else 0), _ptr(gate),
            c_long(gate.stride(0) if gate is not None else 0), c_int(gate_per), c_float(softcap), _stream()))
        return
    attention_flex(q, out, k_cache, v_cache, ctx, seq_pages, page_size, n_heads, n_kv_heads, maps, dk, dv, scale, head_scale,
                   window, chunk, pooled, gate, softcap)


_MAPS_ATTENTION = os.environ.get("LLMI_MAPS_ATTENTION", "mma")      # "generic": the fp32-arithmetic kernel for everything
_MAPS_BLOCKS_PER_SM = int(os.environ.get("LLMI_MAPS_BLOCKS_PER_SM", "3"))


def maps_attention_plan(n_seqs: int, n_pages: int, kv_head_maps: int, window: int, chunk: int, page_size: int,
                        pool: int = 0) -> tuple:
    """(cuts over the positions, pages per cut) of the tensor-core attention for a step of single tokens: cut until
    about three blocks per SM are at work (measured, batch 8 at 4,096 positions: 0.639 ms a step with two, 0.626 with three, 0.628 with four, 0.636 with six).  A query sees at most the pages its window or its block of positions spans.
    Depends on the step's padded shape only, so a recorded step can be replayed."""
    visible = max(n_pages, 1)
    for span in (window, chunk):
        if span > 0:
            visible = min(visible, -(-span // page_size) + 1)
    if pool > 0:       # pages of pooled rows ahead of the window's pages: one row per `pool` positions
        visible += -(-n_pages // pool)
    want = max(1, min(visible, 256, -(-_MAPS_BLOCKS_PER_SM * sm_count() // max(1, n_seqs * kv_head_maps))))
    pps = -(-visible // want)
    return -(-visible // pps), pps


def diff_combine(a: torch.Tensor, lam: float, eps: float, post: float, H: int, dv: int, ctx, out: torch.Tensor) -> None:
    """out = (a1 - lam * a2) / rms(a1 - lam * a2) * post per (token, head); a fp32 [T, H*2*dv] ([head][map][dv])."""
    _need_cuda(a, out)
    T = a.shape[0]
    assert a.dtype == torch.float32 and a.stride(1) == 1 and a.shape[1] == 2 * H * dv and out.shape == (T, H * dv) and out.stride(1) == 1
    _check("diff_combine", lib().llmi_diff_combine(c_int(_dtype_code(out)), _ptr(a), c_long(a.stride(0)), c_float(lam), c_float(eps),
                                                   c_float(post), c_int(H), c_int(dv), _ptr(ctx.tok_seq), _ptr(out),
                                                   c_long(out.stride(0)), c_int(T), _stream()))


# ---------------------------------------------------------------------------------------------
# A short convolution over time with a carried state (csrc/short_conv.cu); plain activations

def conv_add(h: torch.Tensor, w: torch.Tensor, carry: torch.Tensor, ctx, out: torch.Tensor, write_state: bool = True,
             add_input: bool = True) -> None:
    """out = h + conv(h) (or conv(h) alone with ``add_input`` False; ``h`` may be a view of wider rows): per channel a causal convolution over time with the taps ``w`` fp32 [K, C] (tap-major: the
    channels of a tap lie side by side; the oldest tap first); the K-1 inputs ahead of a step's first row come from
    ``carry`` fp32 [slots, >= (K-1)*C], which is then brought up to date."""
    _need_cuda(h, w, carry, out)
    T, C = h.shape
    K = w.shape[0]
    assert h.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, C) and out.dtype == h.dtype
    assert w.dtype == torch.float32 and w.shape == (K, C) and w.is_contiguous()
    assert carry.dtype == torch.float32 and carry.dim() == 2 and carry.stride(1) == 1 and carry.shape[1] >= (K - 1) * C
    assert out.data_ptr() != h.data_ptr()
    _check("conv_add", lib().llmi_conv_add(c_int(_dtype_code(h)), _ptr(h), c_long(h.stride(0)), _ptr(w), _ptr(carry),
                                           c_long(carry.stride(0)), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(ctx.seq_q_start),
                                           _ptr(ctx.seq_slot), _ptr(out), c_long(out.stride(0)), c_int(T), c_int(C), c_int(K),
                                           c_int(1 if add_input else 0), _stream()))
    if write_state and K > 1:
        _check("conv_carry", lib().llmi_conv_carry(c_int(_dtype_code(h)), _ptr(h), c_long(h.stride(0)), _ptr(carry),
                                                   c_long(carry.stride(0)), _ptr(ctx.seq_q_start), _ptr(ctx.seq_kv_len),
                                                   _ptr(ctx.seq_slot), c_int(ctx.n_seqs), c_int(C), c_int(K), _stream()))


def conv_token(h: torch.Tensor, w: torch.Tensor, carry: torch.Tensor, ctx, out: torch.Tensor, write_state: bool = True) -> None:
    """For a step in which every sequence brings one token: out = conv(h) (the input itself not added; fp32 rows, ``h`` may be
    a view of wider rows) and ``carry`` brought up to date — the results of :func:`conv_add` with ``add_input`` False in
    one kernel.  Relies on a slot's state being zero where a sequence has no earlier positions."""
    _need_cuda(h, w, carry, out)
    T, C = h.shape
    K = w.shape[0]
    assert h.dtype == out.dtype == torch.float32 and h.stride(1) == 1 and out.stride(1) == 1 and out.shape == (T, C)
    assert w.dtype == torch.float32 and w.shape == (K, C) and w.is_contiguous()
    assert carry.dtype == torch.float32 and carry.dim() == 2 and carry.stride(1) == 1 and carry.shape[1] >= (K - 1) * C
    _check("conv_token", lib().llmi_conv_token(_ptr(h), c_long(h.stride(0)), _ptr(w), _ptr(carry), c_long(carry.stride(0)),
                                               _ptr(ctx.tok_seq), _ptr(ctx.seq_slot), _ptr(out), c_long(out.stride(0)), c_int(T),
                                               c_int(C), c_int(K), c_int(1 if write_state else 0), _stream()))


def norm_conv_token(x: torch.Tensor, norm_w: torch.Tensor, eps: float, w: torch.Tensor, carry: torch.Tensor, ctx,
                    out: torch.Tensor, write_state: bool = True) -> None:
    """For a step in which every sequence brings one token: out = h + conv(h) with h = rmsnorm(x) (rounded to out's type
    as :func:`rmsnorm` rounds it), and ``carry`` brought up to date — the results of :func:`rmsnorm` + :func:`conv_add`
    in one kernel.  x fp32 [T, C] contiguous; w fp32 [K, C]."""
    _need_cuda(x, norm_w, w, carry, out)
    T, C = x.shape
    K = w.shape[0]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.shape == (T, C) and out.stride(1) == 1
    assert norm_w.dtype == torch.float32 and norm_w.numel() == C and w.dtype == torch.float32 and w.shape == (K, C) and w.is_contiguous()
    assert carry.dtype == torch.float32 and carry.dim() == 2 and carry.stride(1) == 1 and carry.shape[1] >= (K - 1) * C
    _check("norm_conv_token", lib().llmi_norm_conv_token(
        c_int(_dtype_code(out)), _ptr(x), _ptr(norm_w), c_float(eps), _ptr(w), _ptr(carry), c_long(carry.stride(0)),
        _ptr(ctx.tok_seq), _ptr(ctx.seq_slot), _ptr(out), c_long(out.stride(0)), c_int(T), c_int(C), c_int(K),
        c_int(1 if write_state else 0), _stream()))


ACT_RELU2, ACT_GELU = 0, 1
PLAIN_ACTIVATIONS = {"relu2": ACT_RELU2, "gelu": ACT_GELU}
PLAIN_ACTIVATION_MODES = {ACT_RELU2: OUT_RELU2, ACT_GELU: OUT_GELU}      # activation -> the output mode of the products that finish it in their epilogue
_STORE_ACTIVATIONS = {mode: act for act, mode in PLAIN_ACTIVATION_MODES.items()}


def activate(x: torch.Tensor, out: torch.Tensor, act: int = ACT_RELU2) -> None:
    """out = act(x), elementwise (in place if out is x); act: the square of relu, or the exact GELU."""
    _need_cuda(x, out)
    assert x.is_contiguous() and out.is_contiguous() and x.shape == out.shape and x.dtype == out.dtype
    _check("activate", lib().llmi_activate(c_int(_dtype_code(x)), _ptr(x), _ptr(out), c_long(x.numel()), c_int(act), _stream()))


# ---------------------------------------------------------------------------------------------
# Dynamic Tanh, and what a looped span adds to the stream

def dyt(x: torch.Tensor, weight, bias, alpha: float, out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """out[r] = tanh(alpha * x[src]) * weight + bias, src = rows[r] if rows is given else r; x fp32."""
    _need_cuda(x, weight, bias, out, rows)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and bias.dtype == torch.float32
    assert x.is_contiguous() and out.is_contiguous()
    n, W = out.shape
    assert x.shape[1] == W and weight.numel() == W and bias.numel() == W
    _check("dyt", lib().llmi_dyt(c_int(_dtype_code(out)), _ptr(x), _ptr(weight), _ptr(bias), c_float(alpha), _ptr(out),
                                 _ptr(rows), c_int(n), c_int(W), _stream()))


def dyt_add(y: torch.Tensor, weight, bias, alpha: float, x: torch.Tensor, nxt=None, h: torch.Tensor | None = None) -> None:
    """x += tanh(alpha * y) * weight + bias (y, x fp32 [T, W]); with ``nxt = (weight, bias, alpha)`` and ``h`` also
    h = tanh(alpha' * x) * weight' + bias' of the updated x, in h's type."""
    _need_cuda(y, weight, bias, x, h)
    assert y.dtype == torch.float32 and x.dtype == torch.float32 and y.shape == x.shape and y.is_contiguous() and x.is_contiguous()
    T, W = x.shape
    w2, b2, a2 = nxt if nxt is not None else (None, None, 0.0)
    assert (h is None) == (nxt is None)
    if h is not None:
        assert h.shape == x.shape and h.is_contiguous() and w2.dtype == torch.float32 and b2.dtype == torch.float32
    _check("dyt_add", lib().llmi_dyt_add(_ptr(y), _ptr(weight), _ptr(bias), c_float(alpha), _ptr(x),
                                         c_int(_dtype_code(h) if h is not None else 0), _ptr(h), _ptr(w2), _ptr(b2), c_float(a2),
                                         c_int(T), c_int(W), _stream()))


def stream_add(x: torch.Tensor, add: torch.Tensor | None, vec: torch.Tensor | None) -> None:
    """x += add (same shape, optional), then x += vec (one row for all, optional); fp32."""
    _need_cuda(x, add, vec)
    assert x.dtype == torch.float32 and x.is_contiguous()
    T, W = x.shape
    if add is not None:
        assert add.dtype == torch.float32 and add.shape == x.shape and add.is_contiguous()
    if vec is not None:
        assert vec.dtype == torch.float32 and vec.numel() == W and vec.is_contiguous()
    _check("stream_add", lib().llmi_stream_add(_ptr(x), _ptr(add), _ptr(vec), c_int(T), c_int(W), _stream()))


HEADS_MMA_MIN_TOKENS = int(os.environ.get("LLMI_HEADS_MMA_MIN", "1"))      # from here on the per-head products of a step run on the tensor cores (bf16)


def linear_batched(x: torch.Tensor, bx: int, w: torch.Tensor, out: torch.Tensor, by: int, K: int, mode: int = OUT_STORE) -> None:
    """``w.shape[0]`` products in one launch (one per head): out_b (mode) x_b . w[b]^T with x_b = x[:, b*bx : b*bx + K] and
    out_b = out[:, b*by : b*by + N]; w [batch, N, K] contiguous.  fp32 FMA arithmetic for the 32-bit path and for a
    handful of rows; bf16 products of more rows run as tensor-core tiles (bf16 in, fp32 accumulation)."""
    _need_cuda(x, w, out)
    B, N, Kw = w.shape
    M = x.shape[0]
    assert Kw == K and w.is_contiguous() and x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == M and x.dtype == w.dtype
    assert (B - 1) * bx + K <= x.shape[1] and (B - 1) * by + N <= out.shape[1]
    assert out.dtype == (x.dtype if mode == OUT_STORE else torch.float32)
    if (x.dtype == torch.bfloat16 and mode == OUT_STORE and M >= HEADS_MMA_MIN_TOKENS and not _FORCE_SIMT and K % 8 == 0
            and bx % 8 == 0 and by % 2 == 0 and x.stride(0) % 8 == 0 and out.stride(0) % 2 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and out.data_ptr() % 4 == 0):
        _check("linear_heads_mma", lib().llmi_linear_heads_mma(
            _ptr(x), c_long(x.stride(0)), c_long(bx), _ptr(w), _ptr(out), c_long(out.stride(0)), c_long(by), c_int(B), c_int(M),
            c_int(N), c_int(K), _stream()))
        return
    _check("linear_batched", lib().llmi_linear_simt_batched(
        c_int(_dtype_code(x)), _ptr(x), c_long(x.stride(0)), c_long(bx), _ptr(w), c_long(K), c_long(N * K), _ptr(out),
        c_long(out.stride(0)), c_long(by), c_int(B), c_int(M), c_int(N), c_int(K), c_int(mode), _stream()))


# ---------------------------------------------------------------------------------------------
# Latent attention

def latent_prepare(down: torch.Tensor, Q: int, C: int, R: int, wq, wc, eps: float, inv_freq, rot_dims: int, ctx, seq_pages,
                   page_size: int, cache: torch.Tensor, cq: torch.Tensor, write_kv: bool = True) -> None:
    """From the fp32 down-projection rows [query latent Q | latent C | shared key part R]: the RMS-normed query
    latent into ``cq`` (compute type) and the cache row [normed latent | rotated key part] of every token."""
    _need_cuda(down, wq, wc, inv_freq, seq_pages, cache, cq)
    T = down.shape[0]
    assert down.dtype == torch.float32 and down.stride(1) == 1 and down.shape[1] >= Q + C + R
    assert cq.shape == (T, Q) and cq.is_contiguous() and cq.dtype == cache.dtype and cache.is_contiguous()
    assert cache.shape[-1] == C + R and cache.shape[-3] == 1 and wq.dtype == torch.float32 and wc.dtype == torch.float32
    _check("latent_prepare", lib().llmi_latent_prepare(
        c_int(_dtype_code(cq)), _ptr(down), c_long(down.stride(0)), c_int(Q), c_int(C), c_int(R), _ptr(wq), _ptr(wc), c_float(eps),
        _ptr(inv_freq), c_int(rot_dims), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(seq_pages), c_int(seq_pages.stride(0)),
        c_int(page_size), _ptr(cache), _ptr(cq), c_int(T), c_int(1 if write_kv else 0), _stream()))


def latent_q_rotate(q: torch.Tensor, D: int, qa: torch.Tensor, C: int, R: int, H: int, inv_freq, rot_dims: int, ctx) -> None:
    """The part of every head's query that is rotated by position, q[:, h, D:], into qa[:, h, C:]."""
    _need_cuda(q, qa, inv_freq)
    T = q.shape[0]
    assert q.dtype == qa.dtype and q.stride(1) == 1 and qa.stride(1) == 1
    assert q.shape[1] == H * (D + R) and qa.shape == (T, H * (C + R))
    _check("latent_q_rotate", lib().llmi_latent_q_rotate(
        c_int(_dtype_code(q)), _ptr(q), c_long(q.stride(0)), c_int(D), _ptr(qa), c_long(qa.stride(0)), c_int(C), c_int(R), c_int(H),
        _ptr(inv_freq), c_int(rot_dims), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), c_int(T), _stream()))


_LATENT_ATTENTION = os.environ.get("LLMI_LATENT_ATTENTION", "mma")      # "generic": the fp32-arithmetic kernel for everything


_LATENT_BLOCKS_PER_SM = int(os.environ.get("LLMI_LATENT_BLOCKS_PER_SM", "2"))


def latent_attention_plan(ctx, n_tokens: int, n_pages: int, H: int) -> tuple:
    """(cuts over the positions, pages per cut) of the tensor-core latent attention for a step: prompts are not cut;
    a step of single tokens is cut until about two blocks per SM are at work (the kernel keeps one page buffer
    then, so two blocks share an SM; measured, batch 8 at 4,096 positions: 0.853 ms a step with one block per SM, 0.831
    with two, 0.907 with four).  Depends on the step's padded shape
    only, so a recorded step can be replayed."""
    if not ctx.decode:
        return 1, max(n_pages, 1)
    hpb = 1
    while hpb < H and hpb < 16:
        hpb *= 2
    blocks = -(-n_tokens // (16 // hpb)) * -(-H // hpb)
    want = max(1, min(n_pages, 512, -(-_LATENT_BLOCKS_PER_SM * sm_count() // blocks)))
    pps = -(-n_pages // want)
    return -(-n_pages // pps), pps


def attention_latent(qa: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, ctx, seq_pages, page_size: int, H: int, C: int,
                     R: int, scale: float, rt=None) -> None:
    """Causal attention of every token's heads over its sequence's latent rows: scores from all C + R entries of a
    row, context from its first C.  qa [T, H*(C+R)], out [T, H*C].  bf16 sizes that the tensor-core kernel takes go
    there (``rt`` lends the workspace of its cuts); everything else, and the 32-bit path, to the generic kernel."""
    _need_cuda(qa, out, cache, seq_pages)
    T = qa.shape[0]
    assert qa.dtype == out.dtype == cache.dtype and qa.stride(1) == 1 and out.stride(1) == 1 and cache.is_contiguous()
    assert qa.shape[1] == H * (C + R) and out.shape == (T, H * C) and cache.shape[-1] == C + R and cache.shape[-3] == 1
    if (qa.dtype == torch.bfloat16 and rt is not None and _LATENT_ATTENTION == "mma"
            and lib().llmi_attention_latent_mma_supported(c_int(C), c_int(R), c_int(page_size))
            and qa.data_ptr() % 16 == 0 and qa.stride(0) % 8 == 0):
        splits, pps = latent_attention_plan(ctx, T, seq_pages.shape[1], H)
        n_ws = int(lib().llmi_attention_latent_mma_workspace(c_int(T), c_int(H), c_int(C), c_int(splits)))
        ws = rt.scratch("latent_partials", (n_ws,), torch.float32) if n_ws else None
        _check("attention_latent_mma", lib().llmi_attention_latent_mma(
            _ptr(qa), c_long(qa.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(cache), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos),
            _ptr(seq_pages), c_int(seq_pages.stride(0)), c_int(page_size), c_int(T), c_int(H), c_int(C), c_int(R), c_float(scale),
            c_int(splits), c_int(pps), c_int(1 if ctx.decode else 2), _ptr(ws), c_long(n_ws), _stream()))
        return
    _check("attention_latent", lib().llmi_attention_latent(
        c_int(_dtype_code(qa)), _ptr(qa), c_long(qa.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(cache), _ptr(ctx.tok_seq),
        _ptr(ctx.tok_pos), _ptr(seq_pages), c_int(seq_pages.stride(0)), c_int(page_size), c_int(T), c_int(H), c_int(C), c_int(R),
        c_float(scale), _stream()))


# ---------------------------------------------------------------------------------------------
# Gated delta rule

def delta_state_floats(H: int, Hk: int, D: int, Dv: int, taps: int) -> int:
    """fp32 entries of one sequence's state: S [H, D, Dv] and the convolution's last taps-1 inputs."""
    return int(lib().llmi_delta_state_floats(c_int(H), c_int(Hk), c_int(D), c_int(Dv), c_int(taps)))


def delta_step(proj: torch.Tensor, dims, conv_w, a_log, dt_bias, state: torch.Tensor, ctx, prep: torch.Tensor,
               o_raw: torch.Tensor, write_state: bool = True) -> None:
    """The recurrent part of a gated-delta-rule mixer for one step.  ``proj`` fp32 [T, .]: [q | k | v | b | a | gate]
    rows; ``dims = (H, Hk, D, Dv, taps)``; ``state`` [slots, state_floats] fp32 (read, and updated if
    ``write_state``); ``prep`` fp32 [T, 2*Hk*D + H*Dv + 2*H] scratch; ``o_raw`` fp32 [T, H*Dv] receives S^T q."""
    _need_cuda(proj, conv_w, a_log, dt_bias, state, prep, o_raw)
    H, Hk, D, Dv, taps = dims
    T = proj.shape[0]
    n_conv = 2 * Hk * D + H * Dv
    assert proj.dtype == prep.dtype == o_raw.dtype == state.dtype == torch.float32 and proj.stride(1) == 1
    assert proj.shape[1] == n_conv + 2 * H + H * Dv and prep.shape == (T, n_conv + 2 * H) and o_raw.shape == (T, H * Dv)
    assert prep.is_contiguous() and o_raw.is_contiguous() and state.is_contiguous() and conv_w.shape == (n_conv, taps)
    assert conv_w.dtype == torch.float32 and conv_w.is_contiguous() and a_log.numel() == H and dt_bias.numel() == H
    assert state.shape[-1] == delta_state_floats(H, Hk, D, Dv, taps)
    l = lib()
    d = (c_int(H), c_int(Hk), c_int(D), c_int(Dv), c_int(taps))
    _check("delta_prepare", l.llmi_delta_prepare(_ptr(proj), c_long(proj.stride(0)), *d, _ptr(conv_w), _ptr(a_log), _ptr(dt_bias),
                                                 _ptr(state), _ptr(ctx.tok_seq), _ptr(ctx.tok_pos), _ptr(ctx.seq_q_start),
                                                 _ptr(ctx.seq_slot), _ptr(prep), c_long(prep.stride(0)), c_int(T), _stream()))
    if write_state and taps > 1:
        _check("delta_conv_carry", l.llmi_delta_conv_carry(_ptr(proj), c_long(proj.stride(0)), *d, _ptr(state), _ptr(ctx.seq_q_start),
                                                           _ptr(ctx.seq_kv_len), _ptr(ctx.seq_slot), c_int(ctx.n_seqs), _stream()))
    _check("delta_recurrence", l.llmi_delta_recurrence(_ptr(prep), c_long(prep.stride(0)), *d, _ptr(state), _ptr(ctx.seq_q_start),
                                                       _ptr(ctx.seq_slot), _ptr(o_raw), c_long(o_raw.stride(0)), c_int(ctx.n_seqs),
                                                       c_int(1 if write_state else 0), _stream()))


GATE_SILU, GATE_SIGMOID = 0, 1


def delta_finish(o_raw: torch.Tensor, gate: torch.Tensor, weight, eps: float, H: int, Dv: int, ctx, out: torch.Tensor,
                 gate_act: int = GATE_SILU) -> None:
    """out = o / rms(o) * weight * act(gate) per (token, head); o_raw fp32 [T, H*Dv], gate fp32 [T, H*Dv] (a strided
    view), out in the compute type.  ``weight``: [Dv] (one vector for all heads) or [H*Dv]; ``gate_act``: silu or the
    logistic function."""
    _need_cuda(o_raw, gate, weight, out)
    T = o_raw.shape[0]
    assert o_raw.dtype == gate.dtype == weight.dtype == torch.float32 and gate.stride(1) == 1 and out.stride(1) == 1
    assert gate.shape == (T, H * Dv) and out.shape == (T, H * Dv) and weight.numel() in (Dv, H * Dv) and weight.is_contiguous()
    per_head = Dv if (weight.numel() == H * Dv and H > 1) else 0
    _check("delta_finish", lib().llmi_delta_finish(c_int(_dtype_code(out)), _ptr(o_raw), c_long(o_raw.stride(0)), _ptr(gate),
                                                   c_long(gate.stride(0)), _ptr(weight), c_int(per_head), c_int(gate_act),
                                                   c_float(eps), c_int(H), c_int(Dv), _ptr(ctx.tok_seq), _ptr(out),
                                                   c_long(out.stride(0)), c_int(T), _stream()))


# ---------------------------------------------------------------------------------------------
# The delta rule in its general form (csrc/dplr_delta.cu)

def gdelta_prepare(proj: torch.Tensor, H: int, D: int, Dv: int, w2t: torch.Tensor, w0, a_bias, ctx, prep: torch.Tensor,
                   z: torch.Tensor | None = None) -> None:
    """From the fp32 rows [r | k | v | a | gate | low] (H*D, H*D, H*Dv, H*D, H*Dv, R entries) the recurrence's vectors
    [w | p | m] (H*D each) into ``prep``: w = exp(-exp(-1/2) sigmoid(w0 + W2 tanh(low))), p = k / |k| per head,
    m = -sigmoid(a + a_bias) p.  ``w2t``: W2 transposed, fp32 [R, H*D]; ``z`` (optional) fp32 [T, H*D]: W2 tanh(low) made
    by a matrix product beforehand (:func:`tanh_rows`, :func:`linear`)."""
    _need_cuda(proj, w2t, w0, a_bias, prep, z)
    T = proj.shape[0]
    R = w2t.shape[0]
    assert proj.dtype == prep.dtype == w2t.dtype == w0.dtype == a_bias.dtype == torch.float32
    assert proj.stride(1) == 1 and prep.stride(1) == 1 and proj.shape[1] >= 3 * H * D + 2 * H * Dv + R and prep.shape[1] >= 3 * H * D
    assert w2t.shape == (R, H * D) and w2t.is_contiguous() and w0.numel() == H * D and a_bias.numel() == H * D
    assert z is None or (z.dtype == torch.float32 and z.shape == (T, H * D) and z.stride(1) == 1)
    _check("gdelta_prepare", lib().llmi_gdelta_prepare(_ptr(proj), c_long(proj.stride(0)), c_int(H), c_int(D), c_int(Dv), c_int(R),
                                                       _ptr(w2t), _ptr(z), c_long(z.stride(0) if z is not None else 0), _ptr(w0),
                                                       _ptr(a_bias), _ptr(ctx.tok_seq), _ptr(prep), c_long(prep.stride(0)),
                                                       c_int(T), _stream()))


def tanh_rows(src: torch.Tensor, out: torch.Tensor) -> None:
    """out [T, R] (contiguous, any compute type) = tanh(src), src an fp32 view [T, R] with strided rows."""
    _need_cuda(src, out)
    T, R = out.shape
    assert src.dtype == torch.float32 and src.shape == (T, R) and src.stride(1) == 1 and out.is_contiguous()
    _check("tanh_rows", lib().llmi_tanh_rows(c_int(_dtype_code(out)), _ptr(src), c_long(src.stride(0)), _ptr(out), c_int(T), c_int(R),
                                             _stream()))


def dplr_recurrence(proj: torch.Tensor, prep: torch.Tensor, H: int, D: int, Dv: int, state: torch.Tensor, ctx,
                    o_raw: torch.Tensor, write_state: bool = True) -> None:
    """Per head S <- diag(w) S + m (p^T S) + k v^T, o = S^T r over the step's tokens of every sequence.  ``proj`` fp32
    rows with r, k, v at columns 0, H*D, 2*H*D; ``prep`` fp32 rows with w, p, m at 0, H*D, 2*H*D; ``state`` fp32
    [slots, >= H*D*Dv] (S column by column; read, and updated if ``write_state``); ``o_raw`` fp32 [T, H*Dv]."""
    _need_cuda(proj, prep, state, o_raw)
    assert proj.dtype == prep.dtype == state.dtype == o_raw.dtype == torch.float32
    assert proj.stride(1) == 1 and prep.stride(1) == 1 and o_raw.stride(1) == 1 and state.dim() == 2 and state.stride(1) == 1
    assert state.shape[1] >= H * D * Dv and o_raw.shape == (proj.shape[0], H * Dv)
    _check("dplr_recurrence", lib().llmi_dplr_recurrence(
        _ptr(proj), c_long(proj.stride(0)), _ptr(prep), c_long(prep.stride(0)), c_int(H), c_int(D), c_int(Dv), _ptr(state),
        c_long(state.stride(0)), _ptr(ctx.seq_q_start), _ptr(ctx.seq_slot), _ptr(o_raw), c_long(o_raw.stride(0)),
        c_int(ctx.n_seqs), c_int(1 if write_state else 0), _stream()))


# ---------------------------------------------------------------------------------------------
# Routed experts

ROUTE_SOFTMAX_CHOSEN, ROUTE_LOGISTIC_NORMALISED = 0, 1
ROUTE_SOFTMAX_ALL = 2      # scores: the softmax over ALL logits; chosen by score + correction; weights: score * scale, not normalised
ROUTE_MODES = {"softmax_chosen": ROUTE_SOFTMAX_CHOSEN, "logistic_normalised": ROUTE_LOGISTIC_NORMALISED,
               "softmax_all": ROUTE_SOFTMAX_ALL}


def moe_route(logits: torch.Tensor, top: int, ctx, idx: torch.Tensor, wt: torch.Tensor, mode: int = ROUTE_SOFTMAX_CHOSEN,
              n_groups: int = 0, keep: int = 0, experts: int | None = None, correction: torch.Tensor | None = None,
              scale: float = 1.0, identity: int = 0, id_wt: torch.Tensor | None = None) -> None:
    """The ``top`` largest of each row's fp32 logits (ties: the lower index) into ``idx`` int32 [T, top], and the
    softmax over them into ``wt`` fp32 [T, top]; a token row of no sequence gets index -1.  ``mode``
    ROUTE_LOGISTIC_NORMALISED: the scores are logistic(logit) and the weights the chosen scores over their sum (+ 1e-20).
    ``n_groups`` > 1 with ``keep`` < n_groups: only experts of the ``keep`` best of ``n_groups`` equal runs of neighbours
    can be chosen (a run's score: the sum of its two largest scores).  ``experts``: the first columns of ``logits`` that
    are experts (default: all).  ``mode`` ROUTE_SOFTMAX_ALL: the scores are the softmax over all ``experts`` logits, the
    choice goes by score + ``correction`` (fp32 [experts], optional), the weights are the chosen scores times ``scale``;
    the last ``identity`` of the experts hand their input on: such a choice gets index -1 and the token's summed weight
    of them goes to ``id_wt`` fp32 [T] (see :func:`moe_identity_add`)."""
    _need_cuda(logits, idx, wt, correction, id_wt)
    assert correction is None or (correction.dtype == torch.float32 and correction.is_contiguous())
    assert id_wt is None or (id_wt.dtype == torch.float32 and id_wt.is_contiguous() and id_wt.numel() >= logits.shape[0])
    T, E = logits.shape
    E = E if experts is None else int(experts)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and idx.dtype == torch.int32 and wt.dtype == torch.float32
    assert idx.shape == (T, top) and wt.shape == (T, top) and idx.is_contiguous() and wt.is_contiguous()
    _check("moe_route", lib().llmi_moe_route(_ptr(logits), c_long(logits.stride(0)), c_int(E), c_int(top), c_int(mode),
                                             c_int(n_groups), c_int(keep), _ptr(ctx.tok_seq), _ptr(idx), _ptr(wt), c_int(T),
                                             _ptr(correction), c_float(scale), c_int(identity), _ptr(id_wt), _stream()))


def moe_identity_add(h: torch.Tensor, id_wt: torch.Tensor, y: torch.Tensor) -> None:
    """y[t] += id_wt[t] * h[t]: what a token's chosen experts that hand their input on add.  h [T, W] in the compute type
    (row-strided), id_wt fp32 [T], y fp32 [T, W] (row-strided)."""
    _need_cuda(h, id_wt, y)
    T, W = h.shape
    assert h.stride(1) == 1 and y.stride(1) == 1 and y.shape == (T, W) and y.dtype == id_wt.dtype == torch.float32
    _check("moe_identity_add", lib().llmi_moe_identity_add(c_int(_dtype_code(h)), _ptr(h), c_long(h.stride(0)), _ptr(id_wt), _ptr(y),
                                                           c_long(y.stride(0)), c_int(W), c_int(T), _stream()))


def moe_experts_streamed(h: torch.Tensor, w_gate, w_up, w_down, idx, wt, act: int, a: torch.Tensor, y: torch.Tensor,
                         add: bool = False) -> None:
    """y = sum over each token's choices of wt * down_e(act(gate_e h) * up_e h); the weight-streaming form.
    w_gate, w_up [E, F, W], w_down [E, W, F] in h's type; a fp32 [T, top, F] scratch; y fp32 [T, W] (stored, or with ``add`` added to).
    ``w_gate`` None: experts without a gate matrix, down_e(act(up_e h))."""
    _need_cuda(h, w_gate, w_up, w_down, idx, wt, a, y)
    T, W = h.shape
    E, F, _ = w_up.shape
    top = idx.shape[1]
    assert h.stride(1) == 1 and h.dtype == w_up.dtype == w_down.dtype and (w_gate is None or w_gate.dtype == h.dtype)
    assert (w_gate is None or (w_gate.is_contiguous() and w_gate.shape == w_up.shape)) and w_up.is_contiguous() and w_down.is_contiguous() and w_down.shape == (E, W, F)
    assert a.dtype == torch.float32 and a.is_contiguous() and a.numel() >= T * top * F and y.dtype == torch.float32 and y.stride(1) == 1
    l = lib()
    _check("moe_up", l.llmi_moe_up(c_int(_dtype_code(h)), _ptr(h), c_long(h.stride(0)), _ptr(w_gate), _ptr(w_up), c_int(W), c_int(F),
                                   c_int(top), _ptr(idx), _ptr(a), c_int(act), c_int(T), _stream()))
    _check("moe_down", l.llmi_moe_down(c_int(_dtype_code(h)), _ptr(a), _ptr(w_down), c_int(W), c_int(F), c_int(top), _ptr(idx),
                                       _ptr(wt), _ptr(y), c_long(y.stride(0)), c_int(T), c_int(1 if add else 0), _stream()))


MOE_GROUPED_MIN_TOKENS = int(os.environ.get("LLMI_MOE_GROUPED_MIN", "4"))


def moe_grouped_applies(h: torch.Tensor, W: int, F: int, E: int) -> bool:
    """Whether a step's routed experts run as grouped tensor-core tiles (bf16, many tokens) or stream their weights."""
    return bool(h.dtype == torch.bfloat16 and h.shape[0] >= MOE_GROUPED_MIN_TOKENS and W % 8 == 0 and F % 8 == 0 and E <= 256
                and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0 and not _FORCE_SIMT)


def moe_experts_grouped(h: torch.Tensor, w_gate, w_up, w_down, idx, wt, act: int, rt, y: torch.Tensor, add: bool = False,
                        id_wt: torch.Tensor | None = None) -> None:
    """The same result as :func:`moe_experts_streamed` for many tokens: the (token, choice) items are grouped by expert
    and each expert's products run as tensor-core tiles over its rows.  bf16; ``rt`` lends the scratch.  ``id_wt`` (fp32
    [T], optional): id_wt[t] * h[t] joins token t's sum (what :func:`moe_identity_add` adds, without a kernel of its own)."""
    _need_cuda(h, w_gate, w_up, w_down, idx, wt, y, id_wt)
    assert id_wt is None or (id_wt.dtype == torch.float32 and id_wt.is_contiguous() and id_wt.numel() >= h.shape[0])
    T, W = h.shape
    E, F, _ = w_up.shape
    top = idx.shape[1]
    assert h.dtype == w_up.dtype == w_down.dtype == torch.bfloat16 and h.stride(1) == 1
    assert (w_gate is None or (w_gate.dtype == torch.bfloat16 and w_gate.is_contiguous() and w_gate.shape == w_up.shape)) and w_up.is_contiguous() and w_down.is_contiguous() and w_down.shape == (E, W, F)
    assert y.dtype == torch.float32 and y.stride(1) == 1 and idx.is_contiguous() and wt.is_contiguous()
    n_int = int(lib().llmi_moe_group_ints(c_int(T * top), c_int(E)))
    scratch = rt.scratch("experts_groups", (n_int,), torch.int32)
    a_sorted = rt.scratch("experts_act_sorted", (T * top, F), torch.bfloat16)
    y_sorted = rt.scratch("experts_out_sorted", (T * top, W), torch.float32)
    # experts without a gate matrix take the tcgen05 tiles from 1,024 items on: those read the items' input rows in the
    # grouping's order from a buffer of their own
    h_sorted = rt.scratch("experts_in_sorted", (T * top, W), torch.bfloat16) if w_gate is None and T * top >= 1024 else None
    _check("moe_grouped", lib().llmi_moe_grouped(
        _ptr(h), c_long(h.stride(0)), _ptr(w_gate), _ptr(w_up), _ptr(w_down), c_int(W), c_int(F), c_int(E), c_int(top), _ptr(idx),
        _ptr(wt), c_int(act), _ptr(scratch), c_long(n_int), _ptr(a_sorted), _ptr(y_sorted), _ptr(y), c_long(y.stride(0)), c_int(T),
        c_int(1 if add else 0), _ptr(h_sorted), _ptr(tc_scratch(h.device).error), _ptr(id_wt), _stream()))


# ---------------------------------------------------------------------------------------------
# Linear attention with a decay (csrc/decay_recurrence.cu)

def channel_decay(low: torch.Tensor, w2t: torch.Tensor, bias, tau: float, ctx, dec: torch.Tensor, w2: torch.Tensor | None = None) -> None:
    """dec[t, c] = logistic(bias[c] + sum_j w2t[j, c] * low[t, j]) ** (1 / tau), in fp32 (as exp(log_logistic(z) / tau)).
    low fp32 [T, R] (a view of wider rows), w2t fp32 [R, N], bias fp32 [N] or None, dec fp32 [T, N].  ``w2`` (optional): the
    same matrix untransposed, fp32 [N, R]: a handful of tokens read it row by row (the same sums in the same order)."""
    _need_cuda(low, w2t, bias, dec, w2)
    assert w2 is None or (w2.dtype == torch.float32 and w2.is_contiguous() and w2.shape == (w2t.shape[1], w2t.shape[0]))
    T, R = low.shape
    N = w2t.shape[1]
    assert low.dtype == w2t.dtype == dec.dtype == torch.float32 and low.stride(1) == 1 and dec.stride(1) == 1
    assert w2t.shape == (R, N) and w2t.is_contiguous() and dec.shape == (T, N) and (bias is None or (bias.dtype == torch.float32 and bias.numel() == N))
    _check("channel_decay", lib().llmi_channel_decay(_ptr(low), c_long(low.stride(0)), c_int(R), _ptr(w2t), _ptr(w2), _ptr(bias), c_float(tau),
                                                     c_int(N), _ptr(ctx.tok_seq), _ptr(dec), c_long(dec.stride(0)), c_int(T), _stream()))


def rows_silu(x: torch.Tensor) -> None:
    """x = silu(x) in place; x fp32 [T, n], a view of wider rows."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.stride(1) == 1
    _check("rows_activate", lib().llmi_rows_activate(_ptr(x), c_long(x.stride(0)), c_int(x.shape[1]), c_int(x.shape[0]), c_int(0), _stream()))


def decay_recurrence(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, H: int, D: int, Dv: int, state: torch.Tensor, ctx,
                     o_raw: torch.Tensor, dec: torch.Tensor | None = None, head_decay: torch.Tensor | None = None,
                     q_scale: float = 1.0, write_state: bool = True, silu_in: bool = False) -> None:
    """Per sequence and head, over the step's tokens:  S <- diag(w) S + k v^T,  o = q_scale * S^T q.  With ``silu_in`` q, k
    and v pass silu as they are read (for a handful of tokens: no pass of its own over the rows, the same values).  q, k (H*D entries) and
    v (H*Dv) lie in the fp32 rows ``proj`` at the given column offsets; w is ``dec`` fp32 [T, H*D] (a factor per key channel
    and token) or ``head_decay`` fp32 [H] (one constant factor per head).  ``state`` fp32 [slots, >= H*D*Dv] holds S column
    by column and is continued; ``o_raw`` fp32 [T, H*Dv]."""
    _need_cuda(proj, state, o_raw, dec, head_decay)
    T = proj.shape[0]
    assert proj.dtype == state.dtype == o_raw.dtype == torch.float32 and proj.stride(1) == 1 and o_raw.stride(1) == 1
    assert state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= H * D * Dv and o_raw.shape == (T, H * Dv)
    assert (dec is None) != (head_decay is None)
    assert dec is None or (dec.dtype == torch.float32 and dec.shape == (T, H * D) and dec.stride(1) == 1)
    assert head_decay is None or (head_decay.dtype == torch.float32 and head_decay.numel() == H and head_decay.is_contiguous())
    assert max(q_off, k_off) + H * D <= proj.shape[1] and v_off + H * Dv <= proj.shape[1]
    _check("decay_recurrence", lib().llmi_decay_recurrence(
        _ptr(proj), c_long(proj.stride(0)), c_int(q_off), c_int(k_off), c_int(v_off), _ptr(dec),
        c_long(dec.stride(0) if dec is not None else 0), _ptr(head_decay), c_float(q_scale), c_int(H), c_int(D), c_int(Dv),
        _ptr(state), c_long(state.stride(0)), _ptr(ctx.seq_q_start), _ptr(ctx.seq_slot), _ptr(o_raw), c_long(o_raw.stride(0)),
        c_int(ctx.n_seqs), c_int(1 if write_state else 0), c_int(1 if silu_in else 0), _stream()))


# ---------------------------------------------------------------------------------------------
# Joining the branches of a layer (csrc/branch_parts.cu)

def normed_pair(a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor, eps: float, coeff: float, y: torch.Tensor,
                add: bool = False) -> None:
    """y (+)= coeff * (a / rms(a) * wa + b / rms(b) * wb) row by row, rms(v) = sqrt(mean(v^2) + eps); all fp32 [T, W]."""
    _need_cuda(a, wa, b, wb, y)
    T, W = a.shape
    assert a.dtype == b.dtype == y.dtype == wa.dtype == wb.dtype == torch.float32 and b.shape == (T, W) and y.shape == (T, W)
    assert a.stride(1) == 1 and b.stride(1) == 1 and y.stride(1) == 1 and wa.numel() == W and wb.numel() == W
    _check("normed_pair", lib().llmi_normed_pair(_ptr(a), c_long(a.stride(0)), _ptr(wa), _ptr(b), c_long(b.stride(0)), _ptr(wb),
                                                 c_float(eps), c_float(coeff), _ptr(y), c_long(y.stride(0)), c_int(W), c_int(T),
                                                 c_int(1 if add else 0), _stream()))


def stream_axpy_norm(x: torch.Tensor, y: torch.Tensor, m: float, norm_w: torch.Tensor | None = None, eps: float = 0.0,
                     h: torch.Tensor | None = None) -> None:
    """x += m * y (fp32 [T, W], contiguous).  With ``norm_w`` (fp32 [W]) and ``h`` [T, W] (compute type, contiguous): also
    h = norm_w * x / rms(x) of the new x, in the same pass."""
    _need_cuda(x, y, norm_w, h)
    T, W = x.shape
    assert x.dtype == y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape == (T, W)
    assert (norm_w is None) == (h is None)
    if h is not None:
        assert norm_w.dtype == torch.float32 and norm_w.numel() == W and h.shape == (T, W) and h.is_contiguous()
    _check("stream_axpy_norm", lib().llmi_stream_axpy_norm(_ptr(x), _ptr(y), c_float(m), c_int(T), c_int(W), _ptr(norm_w), c_float(eps),
                                                           c_int(_dtype_code(h) if h is not None else 0), _ptr(h), _stream()))
