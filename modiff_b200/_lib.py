"""ctypes binding of libmodiff_b200.so (the C ABI declared in include/modiff_b200.h).

There is no CPU fallback: `lib()` raises if the shared library is missing, and every
wrapper raises `ModiffError` when an entry point returns a non-zero status.
"""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmodiff_b200.so")

IMPL_AUTO, IMPL_SIMT, IMPL_TCGEN05 = 0, 1, 2
MODQ_SCRATCH_BYTES = 64


class ModiffError(RuntimeError):
    pass


class ConvGeom(C.Structure):
    """Mirror of `modiff_conv_geom`."""
    _fields_ = [(n, C.c_int32) for n in (
        "batch", "cin", "cout", "h", "w", "kh", "kw", "stride",
        "pad_t", "pad_l", "pad_b", "pad_r", "split")]

    def key(self):
        return tuple(getattr(self, n) for n, _ in self._fields_)

    def copy(self, **kw):
        g = ConvGeom(*[getattr(self, n) for n, _ in self._fields_])
        for k, v in kw.items():
            setattr(g, k, v)
        return g


class ActSourceStruct(C.Structure):
    """Mirror of `modiff_act_source`."""
    _fields_ = [("x0", C.c_void_p), ("x1", C.c_void_p), ("c0", C.c_int32), ("silu", C.c_int32),
                ("affine", C.c_void_p), ("chan_bias", C.c_void_p)]


class LinearItem(C.Structure):
    """Mirror of `modiff_linear_item`."""
    _fields_ = [("wcodes", C.c_void_p), ("w_scale", C.c_void_p), ("w_corr", C.c_void_p),
                ("o_hat", C.c_void_p), ("cout", C.c_int32), ("with_sum_rows", C.c_int32)]


class GemmBf16Desc(C.Structure):
    """Mirror of `modiff_gemm_bf16_desc`."""
    _fields_ = [("a", C.c_void_p), ("b", C.c_void_p), ("col_scale", C.c_void_p),
                ("bias", C.c_void_p), ("out", C.c_void_p), ("a_parts", C.c_int32),
                ("b_parts", C.c_int32), ("b_batched", C.c_int32), ("kb", C.c_int32),
                ("scale", C.c_float), ("b_rows", C.c_int32)]


_P = C.c_void_p
_G = C.POINTER(ConvGeom)

# name -> (restype, argtypes); one entry per declaration of include/modiff_b200.h
SIGNATURES = {
    "modiff_version": (C.c_int, []),
    "modiff_last_error": (C.c_char_p, []),
    "modiff_device_info": (C.c_int, [C.POINTER(C.c_int)] * 3),
    "modiff_device_status": (C.c_int, [C.POINTER(C.c_int), C.c_int]),
    "modiff_codes_bytes": (C.c_int64, [_G]),
    "modiff_wcodes_bytes": (C.c_int64, [_G, C.c_int]),
    "modiff_out_h": (C.c_int32, [_G]),
    "modiff_out_w": (C.c_int32, [_G]),
    "modiff_wcodes_rows": (C.c_int32, [_G, C.c_int]),
    "modiff_weight_pack": (C.c_int, [_P, _G, C.c_int, C.c_int, _P, _P, _P, _P, _P, _P]),
    "modiff_weight_pack_rounded": (C.c_int, [_P, _P, _P, _P, _G, C.c_int, C.c_int, _P, _P, _P, _P,
                                             _P, _P, _P]),
    "modiff_codes_fill_halo": (C.c_int, [_P, _P, _G, _P]),
    "modiff_asym_bias": (C.c_int, [_P, _P, _P, _P, _P, _P, C.c_int, C.c_int, _P]),
    "modiff_igemm_conv_offset": (C.c_int, [_P, _P, C.c_int, _P, _P, _P, _P, _P, _P, C.c_int, _P, _G,
                                           C.c_int, _P, _P, _P]),
    "modiff_modq": (C.c_int, [_P, _P, _P, _P, _G, C.c_int, C.c_int, _P, _P]),
    "modiff_modq_fixed": (C.c_int, [C.POINTER(ActSourceStruct), _P, _P, _P, _P, _G, C.c_int, C.c_int,
                                    _P]),
    "modiff_modq_geglu": (C.c_int, [_P, C.c_int64, C.c_int, _P, _P, _P, C.c_int, _P, _P]),
    "modiff_modq_ln": (C.c_int, [_P, _P, _P, C.c_float, C.c_int64, C.c_int, _P, _P, _P, C.c_int, _P, _P]),
    "modiff_modq_src": (C.c_int, [C.POINTER(ActSourceStruct), _P, _P, _P, _G, C.c_int, C.c_int, _P,
                                  _P]),
    "modiff_modq_pair": (C.c_int, [C.POINTER(ActSourceStruct), _P, _P, C.c_int, C.c_float, _P, _P, _P,
                                   _P, _G, C.c_int, _P, _P, _P, _P, _G, C.c_int, _P, _P]),
    "modiff_modq_asym": (C.c_int, [C.POINTER(ActSourceStruct), _P, _P, _P, _P, _G, C.c_int, C.c_int,
                                   _P, _P]),
    "modiff_modq_gn": (C.c_int, [C.POINTER(ActSourceStruct), _P, _P, _P, C.c_int, C.c_float, _P, _P,
                                 _P, _P, _G, C.c_int, C.c_int, _P, _P]),
    "modiff_modq_gn_asym": (C.c_int, [C.POINTER(ActSourceStruct), _P, _P, _P, C.c_int, C.c_float, _P,
                                      _P, _P, _P, _P, _G, C.c_int, _P, _P]),
    "modiff_modq_up2": (C.c_int, [_P, _P, _P, _P, _G, C.c_int, C.c_int, _P, _P]),
    "modiff_modq_running": (C.c_int, [C.POINTER(ActSourceStruct), _P, _P, _P, _P, _P, _G, C.c_int,
                                      C.c_int, C.c_int, C.c_double, _P, _P]),
    "modiff_modq_static": (C.c_int, [_P, _P, _P, _P, _G, C.c_int, C.c_int, _P]),
    "modiff_attention_tc": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                      C.c_int, C.c_int, C.c_float, _P]),
    "modiff_linear_group": (C.c_int, [_P, _P, C.c_int, C.c_int, _P, _P, C.c_int, _P]),
    "modiff_igemm_conv": (C.c_int, [_P, _P, C.c_int, _P, _P, _P, _P, C.c_int, _P, _G, C.c_int,
                                    C.c_int, _P, _P]),
    "modiff_igemm_conv_add": (C.c_int, [_P, _P, C.c_int, _P, _P, _P, _P, C.c_int, _G, C.c_int, _P, _P,
                                        _P]),
    "modiff_im2col_codes": (C.c_int, [_P, _P, _G, C.c_int, _P]),
    "modiff_conv_fp32": (C.c_int, [_P, _P, _P, _P, _G, _P]),
    "modiff_bf16_planes_bytes": (C.c_int64, [_G]),
    "modiff_split_bf16": (C.c_int, [_P, _P, _G, _P]),
    "modiff_split_bf16_rows": (C.c_int, [_P, _P, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "modiff_weights_bf16_bytes": (C.c_int64, [_G]),
    "modiff_weights_bf16": (C.c_int, [_P, _P, _P, _P, _G, C.c_int, _P]),
    "modiff_weights_bf16_rounded": (C.c_int, [_P, _P, _P, _P, _P, _G, C.c_int, _P]),
    "modiff_gemm_bf16": (C.c_int, [C.POINTER(GemmBf16Desc), _G, _P]),
    "modiff_softmax_split": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "modiff_attention_small": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_float, _P]),
    "modiff_fake_quant": (C.c_int, [_P, _P, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int,
                                    C.c_int, C.c_int, _P, _P, _P, _P]),
    "modiff_groupnorm_silu": (C.c_int, [_P, _P, C.c_int, _P, _P, _P, _P, _P, _P, C.c_int, C.c_int,
                                        C.c_int, C.c_int, C.c_float, C.c_int, _P]),
    "modiff_avgpool2x": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "modiff_silu": (C.c_int, [_P, _P, C.c_int64, _P]),
    "modiff_layernorm": (C.c_int, [_P, _P, _P, _P, C.c_int64, C.c_int, C.c_float, _P]),
    "modiff_geglu": (C.c_int, [_P, _P, C.c_int64, C.c_int, _P]),
    "modiff_transpose": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "modiff_add": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "modiff_upsample2x": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "modiff_concat_c": (C.c_int, [_P, C.c_int, _P, C.c_int, _P, C.c_int, C.c_int, _P]),
    "modiff_timestep_embedding": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "modiff_ddim_step": (C.c_int, [_P, _P, _P, _P, _P, C.c_int64] + [C.c_float] * 5 + [_P]),
    "modiff_cfg_combine": (C.c_int, [_P, _P, _P, C.c_int64, C.c_float, _P]),
    "modiff_pack_int4": (C.c_int, [_P, _P, C.c_int64, _P]),
    "modiff_unpack_int4": (C.c_int, [_P, _P, C.c_int64, C.c_int, _P]),
    "modiff_quantize_static": (C.c_int, [_P, _P, _P, _G, C.c_int, _P]),
    "modiff_i8_mma_probe": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, _P, _P, _P, _P, _P]),
    "modiff_wait_probe": (C.c_int, [C.c_int64, _P, _P]),
    "modiff_pack_weights_int4": (C.c_int, [_P, _P, _P, C.c_int64, C.c_int64, _P, _P]),
    "modiff_igemm_conv_packed4": (C.c_int, [_P, _P, _P, _P, _P, _P, C.c_int, _G, _P, _P, _P]),
    "modiff_adaround_fake_quant": (C.c_int, [_P, _P, _P, _P, _P, C.c_int64, C.c_int64, C.c_int,
                                             C.c_int, _P]),
    "modiff_attn_codes_bytes": (C.c_int64, [C.c_int] * 5),
    "modiff_attn_quantize": (C.c_int, [_P, _P, _P] + [C.c_int] * 5 + [_P, _P, C.c_int, _P, _P, _P,
                                                                   _P, _P, _P]),
    "modiff_attention_i8": (C.c_int, [_P, _P, _P, _P, _P] + [C.c_int] * 5 + [_P, C.c_float, _P]),
}

_lib = None


def lib():
    """Load the shared library once; fail loudly when it was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ModiffError(
                f"{LIB_PATH} is missing: build it with `python -m modiff_b200.build` "
                "(there is no CPU or PyTorch fallback for the quantised path)")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


# kernels one successful call of an entry point launches (for launch accounting)
KERNELS_PER_CALL = {
    "modiff_weight_pack": 2, "modiff_weight_pack_rounded": 2, "modiff_modq_fixed": 1, "modiff_codes_fill_halo": 1, "modiff_asym_bias": 1, "modiff_igemm_conv_offset": 1, "modiff_modq": 2, "modiff_modq_ln": 2, "modiff_modq_geglu": 2, "modiff_modq_src": 2, "modiff_modq_gn": 2, "modiff_modq_asym": 2, "modiff_modq_running": 3, "modiff_modq_up2": 2, "modiff_modq_gn_asym": 2, "modiff_modq_pair": 2, "modiff_modq_static": 2, "modiff_linear_group": 1, "modiff_attention_tc": 1, "modiff_igemm_conv": 1, "modiff_igemm_conv_add": 1, "modiff_conv_fp32": 1, "modiff_im2col_codes": 1, "modiff_split_bf16": 1, "modiff_split_bf16_rows": 1,
    "modiff_weights_bf16": 1, "modiff_weights_bf16_rounded": 1, "modiff_gemm_bf16": 1, "modiff_softmax_split": 1, "modiff_attention_small": 1,
    "modiff_fake_quant": 2, "modiff_groupnorm_silu": 1, "modiff_silu": 1, "modiff_layernorm": 1, "modiff_geglu": 1, "modiff_transpose": 1, "modiff_add": 1,
    "modiff_upsample2x": 1, "modiff_avgpool2x": 1, "modiff_concat_c": 1, "modiff_timestep_embedding": 1,
    "modiff_ddim_step": 1, "modiff_cfg_combine": 1, "modiff_pack_int4": 1, "modiff_unpack_int4": 1,
    "modiff_quantize_static": 1, "modiff_i8_mma_probe": 1, "modiff_wait_probe": 1,
    "modiff_attn_quantize": 2, "modiff_attention_i8": 1, "modiff_adaround_fake_quant": 1,
    "modiff_pack_weights_int4": 1, "modiff_igemm_conv_packed4": 1,
}
LAUNCHES = [0]        # kernels launched through `call` since import
# Bumped whenever a layer allocates or replaces a device buffer that kernels address directly
# (caches, code planes, scales, packed weights) or a flag is set on a single layer: a captured
# CUDA graph holds those addresses, so it is only replayed while this number is unchanged.
GENERATION = [0]


def bump_generation():
    GENERATION[0] += 1

TIMER = None          # a KernelTimer while per-kernel timing is on


class KernelTimer:
    """Brackets every `call` with CUDA events on the current stream and sums, per entry point,
    device time and the algorithmic bytes the caller declares."""

    def __init__(self):
        self.records = {}
        self.ops = {}         # entry point -> tensor-core operations the callers declared

    def add(self, name, start, end, nbytes, tag=None, nops=0):
        self.records.setdefault(name, []).append((start, end, nbytes))
        if nops:
            self.ops[name] = self.ops.get(name, 0) + nops
        if tag is not None:
            self.records.setdefault((name, tag), []).append((start, end, nbytes))

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, recs in self.records.items():
            if not isinstance(name, str):
                continue
            ms = sum(s.elapsed_time(e) for s, e, _ in recs)
            out[name] = dict(launches=len(recs), ms=ms, bytes=sum(b for _, _, b in recs),
                             ops=self.ops.get(name, 0))
        return out

    def by_tag(self):
        """{(entry point, tag): (launches, ms, bytes)} for calls that carried a tag."""
        torch.cuda.synchronize()
        return {k: (len(r), sum(s.elapsed_time(e) for s, e, _ in r), sum(b for _, _, b in r))
                for k, r in self.records.items() if not isinstance(k, str)}


def call(name, *args, nbytes=0, tag=None, nops=0):
    """Invoke an entry point, raise on a non-zero status, account its launches."""
    fn = getattr(lib(), name)
    if TIMER is None:
        rc = fn(*args)
    else:
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        rc = fn(*args)
        end.record()
        TIMER.add(name, start, end, nbytes, tag, nops)
    if rc != 0:
        check(rc)
    LAUNCHES[0] += KERNELS_PER_CALL.get(name, 0)


def check(rc):
    if rc != 0:
        msg = lib().modiff_last_error().decode(errors="replace")
        raise ModiffError(f"libmodiff_b200 error {rc}: {msg}")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def require_cuda(t, what="tensor"):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ModiffError(
            f"{what} must be a CUDA tensor: the quantised path runs only on the GPU "
            "(no CPU fallback)")
    if t.dtype != torch.float32:
        raise ModiffError(f"{what} must be float32, got {t.dtype}")


def device_status(reset=True):
    s = C.c_int(0)
    check(lib().modiff_device_status(C.byref(s), 1 if reset else 0))
    return s.value


def out_hw(g):
    return lib().modiff_out_h(C.byref(g)), lib().modiff_out_w(C.byref(g))


def measure_i8_peak(mode=1, umma_n=256, iters=4096, repeats=5):
    """Int8 tensor-pipe ceiling of the current device in TOPS: `modiff_i8_mma_probe` on every SM
    (mode 2: every SM pair), operands resident in shared memory, best of `repeats` CUDA-event
    timings after one warm-up launch."""
    sms = C.c_int(0)
    check(lib().modiff_device_info(C.byref(sms), None, None))
    units = sms.value // mode
    m = 128 * mode
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(5)
    a = torch.randint(-127, 128, (units * m, 128), generator=g, dtype=torch.int8).to(dev)
    b = torch.randint(-127, 128, (umma_n, 128), generator=g, dtype=torch.int8).to(dev)
    best = None
    for i in range(repeats + 1):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        call('modiff_i8_mma_probe', mode, umma_n, iters, units, a.data_ptr(), b.data_ptr(), None,
             None, stream_ptr())
        end.record()
        end.synchronize()
        ms = start.elapsed_time(end)
        if i > 0 and (best is None or ms < best):
            best = ms
    if device_status(reset=True):
        raise ModiffError("the int8 probe gave up on a bounded wait")
    ops = units * iters * 4 * 2.0 * m * umma_n * 32
    return ops / (best / 1000.0) / 1e12
