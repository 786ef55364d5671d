"""Host-side mirror of the ``kaio-ops`` quantized entry points over the C ABI.

Names, argument order and meaning follow the Rust functions
(``kaio-ops/src/lib.rs:92-123``); a ``torch.Tensor`` on a CUDA device plays the role of
``GpuBuffer<T>`` (``numel()`` is ``GpuBuffer::len()``), :class:`KaioDevice` the role of
``kaio_runtime::KaioDevice`` (an ordinal plus the stream work is enqueued on).  Like the
reference, every call enqueues asynchronously and returns ``None``; errors raise
:class:`kaio_b200.errors.KaioError` subclasses carrying the reference's message text.

PyTorch is used for device memory and streams only; all arithmetic happens in the CUDA
library.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .errors import from_code

GROUP_SIZE = 128


class KaioDevice:
    """``KaioDevice::new(ordinal)`` (kaio-runtime/src/device.rs:59-115)."""

    def __init__(self, ordinal: int = 0, stream: "torch.cuda.Stream | None" = None):
        self.ordinal = int(ordinal)
        self._stream = stream

    def stream_handle(self) -> int:
        s = self._stream if self._stream is not None else torch.cuda.current_stream(self.ordinal)
        return int(s.cuda_stream)

    def info(self):
        p = torch.cuda.get_device_properties(self.ordinal)
        return {"name": p.name, "compute_capability": (p.major, p.minor), "total_memory": p.total_memory}

    def synchronize(self):
        torch.cuda.synchronize(self.ordinal)


def _buf(t: torch.Tensor, dtype: torch.dtype, what: str):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{what}: expected a torch.Tensor, got {type(t).__name__}")
    if t.dtype != dtype:
        raise TypeError(f"{what}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_cuda:
        raise TypeError(f"{what}: expected a CUDA tensor (there is no CPU fallback)")
    if not t.is_contiguous():
        raise TypeError(f"{what}: expected a contiguous tensor")
    return C.c_void_p(t.data_ptr()), C.c_size_t(t.numel())


def _check(code: int):
    if code != 0:
        raise from_code(code, _lib.load().kaio_b200_last_error().decode("utf-8", "replace"))


def _call(device: KaioDevice, name: str, *args):
    lib = _lib.load()
    with torch.cuda.device(device.ordinal):
        _check(getattr(lib, name)(*args, C.c_void_p(device.stream_handle())))


def last_variant() -> str:
    """Kernel variant the last call on this thread dispatched to."""
    return _lib.load().kaio_b200_last_variant().decode()


def device_status(device: KaioDevice):
    """Synchronise and read the device status block; raises ``DeviceTimeout`` if set."""
    lib = _lib.load()
    code = (C.c_uint32 * 4)()
    with torch.cuda.device(device.ordinal):
        rc = lib.kaio_b200_device_status(C.c_void_p(device.stream_handle()), code)
    _check(rc)
    return list(code)


def selftest_bounded_wait(device: KaioDevice, budget_us: int = 5):
    """Launch the library's one-CTA self-test whose device-side wait runs out after
    ``budget_us`` microseconds; the next :func:`device_status` raises ``DeviceTimeout``."""
    _call(device, "kaio_b200_selftest_bounded_wait", C.c_uint32(budget_us))


def probe_int8_mma_rate(device: KaioDevice, iters: int) -> int:
    """Enqueue the INT8 tensor-pipe rate probe (one CTA per SM, ``iters`` back-to-back
    ``tcgen05.mma kind::i8`` M128 N256 K32 each); returns the integer operations it stands for."""
    ops_count = C.c_uint64(0)
    lib = _lib.load()
    with torch.cuda.device(device.ordinal):
        _check(lib.kaio_b200_probe_int8_mma_rate(C.c_uint32(iters), C.byref(ops_count),
                                                 C.c_void_p(device.stream_handle())))
    return int(ops_count.value)


# ------------------------------------------------------------------ W8A8

def matmul_int8(device, a, b, c, scale, m, n, k):
    """``kaio_ops::matmul_int8`` (kaio-ops/src/matmul_int8_kernel.rs:1468-1512)."""
    _call(device, "kaio_b200_matmul_int8", *_buf(a, torch.int8, "a"), *_buf(b, torch.int8, "b"),
          *_buf(c, torch.float32, "c"), C.c_float(scale), m, n, k)


def matmul_int8_scaled(device, a, b, c, a_scale, w_scale, m, n, k):
    """Extension: per-row x per-column scales."""
    _call(device, "kaio_b200_matmul_int8_scaled", *_buf(a, torch.int8, "a"), *_buf(b, torch.int8, "b"),
          *_buf(c, torch.float32, "c"), *_buf(a_scale, torch.float32, "a_scale"),
          *_buf(w_scale, torch.float32, "w_scale"), m, n, k)


def matmul_int8_acc(device, a, b, acc, m, n, k):
    """Extension: raw s32 accumulators."""
    _call(device, "kaio_b200_matmul_int8_acc", *_buf(a, torch.int8, "a"), *_buf(b, torch.int8, "b"),
          *_buf(acc, torch.int32, "acc"), m, n, k)


# ------------------------------------------------------------------ W4A16

def matmul_tc(device, a, b, c, m, n, k):
    """``kaio_ops::matmul_tc`` (kaio-ops/src/matmul_tc_kernel.rs:1583-1626): f16 x f16 -> f32."""
    _call(device, "kaio_b200_matmul_tc", *_buf(a, torch.float16, "a"), *_buf(b, torch.float16, "b"),
          *_buf(c, torch.float32, "c"), m, n, k)


def matmul_tc_f16out(device, a, b, c, m, n, k):
    """Extension: ``matmul_tc`` with the accumulator narrowed to f16 (``c`` float16)."""
    _call(device, "kaio_b200_matmul_tc_f16out", *_buf(a, torch.float16, "a"), *_buf(b, torch.float16, "b"),
          *_buf(c, torch.float16, "c"), m, n, k)


def dequantize_int4(device, b_packed, scales, w, k, n, group_size=GROUP_SIZE):
    """Extension: packed s4 weights + f16 group scales -> f16 ``[k, n]`` row-major with the
    reference's rounding (``f16(q) * f16(scale)`` in f16): the first step of ``matmul_int4`` for
    large ``m``, on its own, for callers that reuse the dequantised weights within a step."""
    _call(device, "kaio_b200_dequantize_int4", *_buf(b_packed, torch.int32, "b_packed"),
          *_buf(scales, torch.float16, "scales"), *_buf(w, torch.float16, "w"), k, n, group_size)


def matmul_tc_async(device, a, b, c, m, n, k):
    """``kaio_ops::matmul_tc_async`` (kaio-ops/src/matmul_tc_async_kernel.rs): same contract."""
    _call(device, "kaio_b200_matmul_tc_async", *_buf(a, torch.float16, "a"), *_buf(b, torch.float16, "b"),
          *_buf(c, torch.float32, "c"), m, n, k)


def matmul_int4(device, a, b_packed, scales, c, m, n, k, group_size):
    """``kaio_ops::matmul_int4`` (kaio-ops/src/matmul_int4_kernel.rs:2126-2171).

    ``b_packed`` is an int32 tensor holding the u32 words (torch has no uint32 arithmetic; the
    bits are what matters).  ``c`` float32 selects the reference form, float16 the extension.
    """
    name = "kaio_b200_matmul_int4" if c.dtype == torch.float32 else "kaio_b200_matmul_int4_f16out"
    _call(device, name, *_buf(a, torch.float16, "a"), *_buf(b_packed, torch.int32, "b_packed"),
          *_buf(scales, torch.float16, "scales"), *_buf(c, c.dtype if c.dtype in (torch.float32, torch.float16)
                                                        else torch.float32, "c"),
          m, n, k, group_size)


def matmul_int4_allgather(device, a, b_packed_shard, scales_shard, out_ptrs, out_numel, world, rank,
                          m, n_total, k, group_size=GROUP_SIZE):
    """Extension: this rank's column shard of a W4A16 GEMM, stored by the kernel into every rank's
    f16 ``[m, n_total]`` buffer.  ``out_ptrs`` are ``world`` device addresses as mapped in this
    process (e.g. ``torch.distributed._symmetric_memory`` ``buffer_ptrs``)."""
    arr = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in out_ptrs])
    _call(device, "kaio_b200_matmul_int4_allgather", *_buf(a, torch.float16, "a"),
          *_buf(b_packed_shard, torch.int32, "b_packed_shard"), *_buf(scales_shard, torch.float16, "scales_shard"),
          C.cast(arr, C.c_void_p), C.c_size_t(out_numel), world, rank, m, n_total, k, group_size)


def matmul_int4_allgather_multicast(device, a, b_packed_shard, scales_shard, out_ptrs, out_numel, multicast_out,
                                    world, rank, m, n_total, k, group_size=GROUP_SIZE):
    """Extension: :func:`matmul_int4_allgather` whose large-``m`` kernel writes each output block once
    through ``multicast_out``, the NVLink multicast address of the ``[m, n_total]`` output
    (``multimem.st``; the switch delivers it to every rank)."""
    arr = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in out_ptrs])
    _call(device, "kaio_b200_matmul_int4_allgather_multicast", *_buf(a, torch.float16, "a"),
          *_buf(b_packed_shard, torch.int32, "b_packed_shard"), *_buf(scales_shard, torch.float16, "scales_shard"),
          C.cast(arr, C.c_void_p), C.c_size_t(out_numel), C.c_void_p(int(multicast_out)), world, rank, m, n_total,
          k, group_size)


def allgather_cols(device, shard, out, m, n_total, world, nccl_comm):
    """Extension: NCCL all-gather of ``[m, n_total/world]`` column shards into the row-major
    ``[m, n_total]`` ``out`` on every rank, through the C ABI.  ``nccl_comm`` is the raw
    ``ncclComm_t`` address of the ranks' communicator."""
    if shard.dtype != out.dtype or shard.dtype not in (torch.float16, torch.float32):
        raise TypeError("allgather_cols: shard and out must both be float16 or float32")
    _call(device, "kaio_b200_allgather_cols", *_buf(shard, shard.dtype, "shard"), *_buf(out, out.dtype, "out"),
          m, n_total, shard.element_size(), world, C.c_void_p(int(nccl_comm)))


def matmul_int4_peer_partials(device, a, b_packed, scales, slot_ptrs, slot_numel, world, rank, scatter,
                              m, n, k, group_size=GROUP_SIZE):
    """Extension: this rank's K shard of a W4A16 GEMM; the f32 partial ``[m, n]`` is stored by the
    kernel into slot ``rank`` of the ranks' staging buffers (``slot_ptrs``: ``world`` device
    addresses as mapped in this process, each f32 ``[world][m][cols]``).  ``scatter=False``: the
    whole partial to every rank (``cols = n``); ``scatter=True``: column block ``d`` to rank ``d``
    only (``cols = n / world``)."""
    arr = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in slot_ptrs])
    _call(device, "kaio_b200_matmul_int4_peer_partials", *_buf(a, torch.float16, "a"),
          *_buf(b_packed, torch.int32, "b_packed"), *_buf(scales, torch.float16, "scales"),
          C.cast(arr, C.c_void_p), C.c_size_t(slot_numel), world, rank, 1 if scatter else 0, m, n, k, group_size)


def sum_partials_f32(device, slots, world, rows, cols, out_ptrs, out_numel, out_ld, out_col0=0):
    """Extension: ``out_d[row, out_col0 + c] = sum_s slots[s][row][c]`` (ascending ``s``) for every
    destination address in ``out_ptrs`` (f32 buffers with row stride ``out_ld``, possibly peer
    memory)."""
    arr = (C.c_void_p * len(out_ptrs))(*[C.c_void_p(int(p)) for p in out_ptrs])
    _call(device, "kaio_b200_sum_partials_f32", *_buf(slots, torch.float32, "slots"), world, rows, cols,
          C.cast(arr, C.c_void_p), len(out_ptrs), C.c_size_t(out_numel), out_ld, out_col0)


def sum_partials_f32_multicast(device, slots, world, rows, cols, multicast_out, out_numel, out_ld, out_col0=0):
    """Extension: the same sum stored once through ``multicast_out``, an address of an NVLink
    multicast object every rank's output buffer is bound to (``multimem.st``; the switch delivers
    the vector to all ranks)."""
    _call(device, "kaio_b200_sum_partials_f32_multicast", *_buf(slots, torch.float32, "slots"), world, rows, cols,
          C.c_void_p(int(multicast_out)), C.c_size_t(out_numel), out_ld, out_col0)


def matmul_int4_silu_gate(device, x, b_packed, scales, act, gu_scratch, m, cols, k, group_size=GROUP_SIZE):
    """Extension: ``act[m, cols] = silu(x W_gate) * (x W_up)`` from W4A16 weights ``[k, 2*cols]`` whose
    columns alternate in blocks of 64 between ``W_gate`` and ``W_up`` (see
    :func:`kaio_b200.ffn.interleave_gate_up`); the activation runs in the GEMM's epilogue for m > 512."""
    if gu_scratch is None:
        scratch = (C.c_void_p(None), C.c_size_t(0))
    else:
        scratch = _buf(gu_scratch, torch.float16, "gu_scratch")
    _call(device, "kaio_b200_matmul_int4_silu_gate", *_buf(x, torch.float16, "x"),
          *_buf(b_packed, torch.int32, "b_packed"), *_buf(scales, torch.float16, "scales"),
          *_buf(act, torch.float16, "act"), *scratch, m, cols, k, group_size)


def allreduce_multimem_f32(device, multicast_in, multicast_out, numel, rows, cols, ld, col0):
    """Extension: this rank's column block ``[col0, col0 + cols)`` of an in-switch all-reduce
    (``multimem.ld_reduce`` + ``multimem.st``) over multicast addresses of symmetric buffers."""
    _call(device, "kaio_b200_allreduce_multimem_f32", C.c_void_p(int(multicast_in)), C.c_void_p(int(multicast_out)),
          C.c_size_t(numel), rows, cols, ld, col0)


# ------------------------------------------------------------------ fused QKV

def qkv_project_int8(device, x, w_q, w_k, w_v, scale_q, scale_k, scale_v, q_out, k_out, v_out, m, n, k):
    """``kaio_ops::qkv_project_int8`` (kaio-ops/src/qkv_project_int8_kernel.rs:2008-2064).

    Scalar scales select the reference form; float32 tensors of length ``n`` the per-column
    extension.
    """
    if isinstance(scale_q, torch.Tensor):
        sq, sl = _buf(scale_q, torch.float32, "scale_q")
        sk, _ = _buf(scale_k, torch.float32, "scale_k")
        sv, _ = _buf(scale_v, torch.float32, "scale_v")
        sl = C.c_size_t(min(scale_q.numel(), scale_k.numel(), scale_v.numel()))
        _call(device, "kaio_b200_qkv_project_int8_colscale", *_buf(x, torch.float16, "x"),
              *_buf(w_q, torch.int8, "w_q"), *_buf(w_k, torch.int8, "w_k"), *_buf(w_v, torch.int8, "w_v"),
              sq, sk, sv, sl, *_buf(q_out, torch.float16, "q_out"), *_buf(k_out, torch.float16, "k_out"),
              *_buf(v_out, torch.float16, "v_out"), m, n, k)
        return
    _call(device, "kaio_b200_qkv_project_int8", *_buf(x, torch.float16, "x"),
          *_buf(w_q, torch.int8, "w_q"), *_buf(w_k, torch.int8, "w_k"), *_buf(w_v, torch.int8, "w_v"),
          C.c_float(scale_q), C.c_float(scale_k), C.c_float(scale_v),
          *_buf(q_out, torch.float16, "q_out"), *_buf(k_out, torch.float16, "k_out"),
          *_buf(v_out, torch.float16, "v_out"), m, n, k)


def qkv_project_w8a8(device, x, w_q, w_k, w_v, scale_q, scale_k, scale_v, q_out, k_out, v_out, m, n, k):
    """Extension: the W8A8 fused QKV projection -- ``x`` (f16) quantised per row to s8 on the fly,
    s32 accumulation on the INT8 tensor pipe, per-row x per-column scales, f16 outputs.
    ``scale_*`` are float32 tensors of length ``n``."""
    sq, _ = _buf(scale_q, torch.float32, "scale_q")
    sk, _ = _buf(scale_k, torch.float32, "scale_k")
    sv, _ = _buf(scale_v, torch.float32, "scale_v")
    sl = C.c_size_t(min(scale_q.numel(), scale_k.numel(), scale_v.numel()))
    _call(device, "kaio_b200_qkv_project_w8a8", *_buf(x, torch.float16, "x"),
          *_buf(w_q, torch.int8, "w_q"), *_buf(w_k, torch.int8, "w_k"), *_buf(w_v, torch.int8, "w_v"),
          sq, sk, sv, sl, *_buf(q_out, torch.float16, "q_out"), *_buf(k_out, torch.float16, "k_out"),
          *_buf(v_out, torch.float16, "v_out"), m, n, k)


def qkv_project_int4(device, x, w_q_packed, w_k_packed, w_v_packed, scales_q, scales_k, scales_v,
                     q_out, k_out, v_out, m, n, k, group_size):
    """``kaio_ops::qkv_project_int4`` (kaio-ops/src/qkv_project_int4_kernel.rs:1495-1555)."""
    _call(device, "kaio_b200_qkv_project_int4", *_buf(x, torch.float16, "x"),
          *_buf(w_q_packed, torch.int32, "w_q_packed"), *_buf(w_k_packed, torch.int32, "w_k_packed"),
          *_buf(w_v_packed, torch.int32, "w_v_packed"), *_buf(scales_q, torch.float16, "scales_q"),
          *_buf(scales_k, torch.float16, "scales_k"), *_buf(scales_v, torch.float16, "scales_v"),
          *_buf(q_out, torch.float16, "q_out"), *_buf(k_out, torch.float16, "k_out"),
          *_buf(v_out, torch.float16, "v_out"), m, n, k, group_size)


# ------------------------------------------------------------------ quantisers

def quantize_rows_int8(device, x, q, scale, m, k):
    """Per-row symmetric INT8 quantiser (``derive_scale`` + ``quantize`` of
    examples/int8_matmul/src/main.rs:41-61, applied per row)."""
    _call(device, "kaio_b200_quantize_rows_int8", *_buf(x, torch.float32, "x"), *_buf(q, torch.int8, "q"),
          *_buf(scale, torch.float32, "scale"), m, k)


def quantize_pack_int4(device, w, packed, scales, k, n, group_size=GROUP_SIZE):
    """Group-wise INT4 quantiser + packer (``quantize_gptq_lite`` + ``pack_s4_weights`` of
    examples/int4_matmul/src/main.rs:48-99)."""
    _call(device, "kaio_b200_quantize_pack_int4", *_buf(w, torch.float32, "w"),
          *_buf(packed, torch.int32, "packed"), *_buf(scales, torch.float16, "scales"), k, n, group_size)


# ------------------------------------------------------------------ gated activation

def silu_gate_f32(device, x, gate, out, n):
    """The ``fused_silu_gate`` user kernel (examples/fused_silu_gate/src/main.rs:13-21):
    ``out[i] = x[i] * sigmoid(x[i]) * gate[i]`` on f32."""
    _call(device, "kaio_b200_silu_gate_f32", *_buf(x, torch.float32, "x"), *_buf(gate, torch.float32, "gate"),
          *_buf(out, torch.float32, "out"), n)


def silu_gate_f16(device, x, gate, out, rows, cols, x_ld=None, gate_ld=None, out_ld=None):
    """The same on f16 ``[rows, cols]`` matrices with row strides (f32 arithmetic, one rounding);
    not in the reference.  ``x`` and ``gate`` may be views into one ``[rows, 2*cols]`` buffer."""
    _call(device, "kaio_b200_silu_gate_f16", *_buf(x, torch.float16, "x"), *_buf(gate, torch.float16, "gate"),
          *_buf(out, torch.float16, "out"), rows, cols, x_ld or cols, gate_ld or cols, out_ld or cols)


# ------------------------------------------------------------------ attention

def attention_tc(device, q, k, v, out, seq_q, seq_k, d_k, d_v):
    """``kaio_ops::attention_tc`` (kaio-ops/src/attention_tc_kernel.rs:2240-2254)."""
    _call(device, "kaio_b200_attention_tc", *_buf(q, torch.float16, "q"), *_buf(k, torch.float16, "k"),
          *_buf(v, torch.float16, "v"), *_buf(out, torch.float32, "out"), seq_q, seq_k, d_k, d_v, 0)


def attention_tc_causal(device, q, k, v, out, seq_q, seq_k, d_k, d_v):
    """``kaio_ops::attention_tc_causal`` (kaio-ops/src/attention_tc_kernel.rs:2257-2271)."""
    _call(device, "kaio_b200_attention_tc", *_buf(q, torch.float16, "q"), *_buf(k, torch.float16, "k"),
          *_buf(v, torch.float16, "v"), *_buf(out, torch.float32, "out"), seq_q, seq_k, d_k, d_v, 1)


def attention_mha_f16(device, q, k, v, out, batch, heads, seq_q, seq_k, head_dim, row_stride, causal):
    """Extension: batched multi-head attention on ``[batch*seq, heads*head_dim]`` f16 buffers."""
    _call(device, "kaio_b200_attention_mha_f16", *_buf(q, torch.float16, "q"), *_buf(k, torch.float16, "k"),
          *_buf(v, torch.float16, "v"), *_buf(out, torch.float16, "out"), batch, heads, seq_q, seq_k,
          head_dim, row_stride, 1 if causal else 0)
