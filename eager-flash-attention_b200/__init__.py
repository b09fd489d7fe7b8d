"""Python host side of the B200 tensor-parallel attention block.

A thin ctypes layer over ``libefa_b200.so`` (the C ABI of ``include/efa_b200.h``) that mirrors the
host interface of eager-flash-attention for this path, name for name:

* ``make_params`` / ``attn_check_params`` / ``blocks_per_tile``  (attn_main.cuh:18-22,68)
* ``flash_attn_tc_forward`` / ``flash_attn_tc_combine`` / ``flash_attn_tc_check_params``
  (flash_attn_tc.cuh:45-60)
* ``project``  (attn_main.cuh:62-65)
* ``make_ctx`` / ``destroy_ctx``  (attn_main.cuh:43-44)
* ``run_mode`` / ``mode_name`` / ``parse_mode``  (run_drivers.cuh:19-26)

All arithmetic happens in the CUDA library. There is no host fallback: if the shared library is
missing, or no sm_100 device is present, the calls raise.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
# EFA_B200_LIB names another build of the same library (a debug build, say); the default is the one beside this file.
LIB_PATH = os.environ.get("EFA_B200_LIB") or os.path.join(_HERE, "libefa_b200.so")

F32, F16 = 0, 1
MODE_ATTN, MODE_ATTN_TILED, MODE_MEGATRON, MODE_SYNC, MODE_OVERLAP, MODE_STREAM, MODE_COMM = range(7)
MODE_NAMES = ("attn", "attn_tiled", "megatron", "sync", "overlap", "stream", "comm")
REDUCE_NCCL, REDUCE_P2P, REDUCE_NVLS, REDUCE_PULL = 0, 1, 2, 3
ROWS_AUTO, ROWS_ASCENDING, ROWS_DESCENDING, ROWS_MIXED = 0, 1, 2, 3
WIRE_AUTO, WIRE_F16, WIRE_F32 = 0, 1, 2
RECIPE_REF, RECIPE_NORMAL = 0, 1


class EfaError(RuntimeError):
    """A call into the CUDA library failed; the message is efa_last_error()."""


class FlashParams(C.Structure):
    """FlashAttnTCParams (flash_attn_tc.cuh:16-23)."""
    _fields_ = [("S", C.c_int), ("d_h", C.c_int), ("H_local", C.c_int), ("split", C.c_int),
                ("causal", C.c_int), ("scale", C.c_float)]


class FlashPartials(C.Structure):
    """FlashAttnTCPartials (flash_attn_tc.cuh:29-34); the pointers are device addresses."""
    _fields_ = [("O_part", C.c_void_p), ("m_part", C.c_void_p), ("l_part", C.c_void_p), ("rows", C.c_int)]


class Params(C.Structure):
    """AttnParams (attn_defs.cuh:70-84) for the fp16 data path."""
    _fields_ = [("S", C.c_int), ("d", C.c_int), ("H", C.c_int), ("R", C.c_int),
                ("H_local", C.c_int), ("d_h", C.c_int), ("d_local", C.c_int),
                ("tile", C.c_int), ("num_tiles", C.c_int),
                ("nbuf", C.c_int), ("split", C.c_int), ("causal", C.c_int),
                ("skip_proj", C.c_int), ("skip_comm", C.c_int), ("reduce", C.c_int), ("group_tiles", C.c_int),
                ("proj_f32", C.c_int), ("row_order", C.c_int), ("reduce_ctas", C.c_int), ("band_rows", C.c_int),
                ("reserve_sms", C.c_int), ("trace", C.c_int), ("wire", C.c_int), ("debug_target_bias", C.c_int), ("flash_tc", FlashParams)]


_BARRIER_FN = C.CFUNCTYPE(C.c_int, C.c_void_p)
_MAX_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_double))
_BCAST_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int)
_GATHER_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)


class WorldStruct(C.Structure):
    _fields_ = [("user", C.c_void_p), ("rank", C.c_int), ("size", C.c_int), ("local_device", C.c_int),
                ("barrier", _BARRIER_FN), ("allreduce_max_f64", _MAX_FN),
                ("bcast_bytes", _BCAST_FN), ("allgather_bytes", _GATHER_FN)]


class Weights(C.Structure):
    """Weights (attn_main.cuh:7-12): device pointers of this rank's fp16 Q, K, V and W_O slice."""
    _fields_ = [("Qh", C.c_void_p), ("Kh", C.c_void_p), ("Vh", C.c_void_p), ("W_O", C.c_void_p)]


class StreamGroup(C.Structure):
    """efa_stream_group: tiles [first_tile, first_tile + ntiles) share one projection and one AllReduce."""
    _fields_ = [("first_tile", C.c_int), ("ntiles", C.c_int)]


class RunStats(C.Structure):
    _fields_ = [("wall_ms", C.c_double), ("attn_kernel_ms", C.c_float), ("proj_ms", C.c_float),
                ("kernel_launches", C.c_int)]


# Every symbol include/efa_b200.h declares, with its ctypes signature.
_SIGNATURES = {
    "efa_abi_version": (C.c_int, []),
    "efa_last_error": (C.c_char_p, []),
    "efa_flash_attn_tc_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                            C.POINTER(FlashPartials), C.c_int, C.c_int,
                                            C.POINTER(FlashParams), C.c_void_p, C.c_void_p, C.c_int]),
    "efa_flash_attn_tc_forward_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                                    C.c_int, C.c_int, C.POINTER(FlashParams), C.c_void_p]),
    "efa_flash_attn_tc_noalloc_status": (C.c_int, [C.POINTER(C.c_int), C.c_int]),
    "efa_flash_attn_tc_combine": (C.c_int, [C.POINTER(FlashPartials), C.c_void_p, C.c_int, C.c_int, C.c_int,
                                            C.POINTER(FlashParams), C.c_void_p]),
    "efa_flash_attn_tc_check_params": (C.c_char_p, [C.POINTER(FlashParams), C.c_int]),
    "efa_convert_f32_to_f16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "efa_project_f16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "efa_compute_qkv_f16": (C.c_int, [C.c_void_p] * 7 + [C.c_int] * 4 + [C.c_void_p]),
    "efa_kernel_status": (C.c_int, [C.POINTER(C.c_int)]),
    "efa_kernel_status_reset": (C.c_int, []),
    "efa_mode_name": (C.c_char_p, [C.c_int]),
    "efa_parse_mode": (C.c_int, [C.c_char_p]),
    "efa_make_params": (C.c_int, [C.POINTER(Params), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "efa_attn_check_params": (C.c_char_p, [C.POINTER(Params)]),
    "efa_blocks_per_tile": (C.c_int, [C.POINTER(Params)]),
    "efa_stream_plan": (C.c_int, [C.POINTER(Params), C.POINTER(StreamGroup), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "efa_stream_row_blocks": (C.c_int, [C.POINTER(Params), C.POINTER(C.c_short), C.c_int]),
    "efa_ctx_set_wait_limit_ms": (C.c_int, [C.c_void_p, C.c_double, C.c_double]),
    "efa_nvls_output": (C.c_int, [C.c_void_p, C.POINTER(Params), C.POINTER(C.c_void_p)]),
    "efa_world_selftest": (C.c_int, [C.POINTER(WorldStruct)]),
    "efa_make_ctx": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(WorldStruct), C.c_int, C.c_int]),
    "efa_destroy_ctx": (C.c_int, [C.c_void_p]),
    "efa_fill_host_inputs": (C.c_int, [C.POINTER(Params), C.c_int, C.c_int, C.c_int,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "efa_run_mode": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(Weights), C.c_void_p, C.POINTER(Params), C.POINTER(RunStats)]),
    "efa_run_mode_residual": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(Weights), C.c_void_p, C.c_void_p, C.POINTER(Params),
                                        C.POINTER(RunStats)]),
    "efa_run_mode_host": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.POINTER(Params), C.POINTER(RunStats)]),
    "efa_run_mode_host_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_int, C.c_int, C.POINTER(Params), C.POINTER(RunStats)]),
}
EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def lib() -> C.CDLL:
    """Load libefa_b200.so (built by ``make -C csrc`` / ``__graft_entry__.build()``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise EfaError(f"{LIB_PATH} is missing: build it with `make -C {_HERE}/csrc` "
                           "(there is no fallback implementation)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)      # raises AttributeError when the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().efa_last_error().decode("utf-8", "replace")


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise EfaError(f"{what} failed ({rc}): {last_error()}")


def _ptr(x) -> Optional[int]:
    """Device/host address of a torch tensor, a numpy array, an int, or None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)!r}")


def _stream(stream) -> Optional[int]:
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream   # torch.cuda.Stream


# ------------------------------------------------------------------------------------------------
# Parameters
# ------------------------------------------------------------------------------------------------
def make_params(S: int, d: int, H: int, tile: int, nbuf: int = 2, split: int = 1, causal: int = 0,
                world_size: int = 1) -> Params:
    """make_params (attn_main.cu:35-60): d_h = d / H, H_local = H / R, scale = 1 / sqrt(d_h)."""
    p = Params()
    _check(lib().efa_make_params(C.byref(p), S, d, H, tile, nbuf, split, int(bool(causal)), world_size), "make_params")
    return p


def attn_check_params(p: Params) -> Optional[str]:
    """attn_check_params (attn_main.cu:62-74): None if runnable, else the reason."""
    why = lib().efa_attn_check_params(C.byref(p))
    return None if why is None else why.decode()


def flash_attn_tc_check_params(fp: FlashParams, q_rows: int) -> Optional[str]:
    why = lib().efa_flash_attn_tc_check_params(C.byref(fp), q_rows)
    return None if why is None else why.decode()


def blocks_per_tile(p: Params) -> int:
    """blocks_per_tile (attn_main.cu:275-280): (tile / 64) * H_local * split."""
    return lib().efa_blocks_per_tile(C.byref(p))


def stream_plan(p: Params):
    """Launch plan of stream mode: ([(first_tile, ntiles), ...] in the order the groups are waited for, band_rows,
    descending). Host arithmetic."""
    groups = (StreamGroup * max(1, p.num_tiles))()
    band, desc = C.c_int(0), C.c_int(0)
    n = lib().efa_stream_plan(C.byref(p), groups, p.num_tiles, C.byref(band), C.byref(desc))
    if n < 0:
        raise EfaError(f"stream_plan failed: {last_error()}")
    return [(groups[i].first_tile, groups[i].ntiles) for i in range(n)], band.value, bool(desc.value)


def stream_row_blocks(p: Params):
    """Order of the 256-row blocks of stream mode's attention launch when it is neither first-to-last nor
    last-to-first (ROWS_MIXED); an empty list otherwise."""
    cap = (p.S + 255) // 256
    buf = (C.c_short * max(1, cap))()
    n = lib().efa_stream_row_blocks(C.byref(p), buf, cap)
    if n < 0:
        raise EfaError(f"stream_row_blocks failed: {last_error()}")
    return [buf[i] for i in range(n)]


def mode_name(mode: int) -> str:
    return lib().efa_mode_name(mode).decode()


def parse_mode(s: str) -> int:
    return lib().efa_parse_mode(s.encode())


# ------------------------------------------------------------------------------------------------
# Kernel launch interface
# ------------------------------------------------------------------------------------------------
def flash_attn_tc_forward(Q, K, V, O, part: Optional[FlashPartials], q_start: int, q_rows: int,
                          fp: FlashParams, stream=None, tile_counters=None, tile_rows: int = 0,
                          o_dtype: int = F16) -> None:
    """flash_attn_tc_forward (flash_attn_tc.cuh:45-50). Asynchronous on ``stream``."""
    rc = lib().efa_flash_attn_tc_forward(_ptr(Q), _ptr(K), _ptr(V), _ptr(O), o_dtype,
                                         C.byref(part) if part is not None else None,
                                         q_start, q_rows, C.byref(fp), _stream(stream),
                                         _ptr(tile_counters), tile_rows)
    _check(rc, "flash_attn_tc_forward")


STATIC_SCRATCH_BYTES = 8 << 20


def flash_attn_tc_forward_noalloc(Q, K, V, O, q_start: int, q_rows: int, fp: FlashParams, stream=None,
                                  o_dtype: int = F16) -> None:
    """Split-KV attention and merge in one call, for callers that cannot allocate device memory when
    they call (a memory pool owns the GPU, or an allocation's device-wide synchronisation is not
    acceptable): the partials live in a fixed STATIC_SCRATCH_BYTES array inside the library. Shapes
    whose partials do not fit are rejected. Calls share that array, so do not let two overlap on the
    GPU; make the first call on a device outside stream capture."""
    rc = lib().efa_flash_attn_tc_forward_noalloc(_ptr(Q), _ptr(K), _ptr(V), _ptr(O), o_dtype, q_start, q_rows,
                                                 C.byref(fp), _stream(stream))
    _check(rc, "flash_attn_tc_forward_noalloc")


def flash_attn_tc_noalloc_status(reset: bool = False) -> Sequence[int]:
    """(code, block, site, 0) of the kernels launched by flash_attn_tc_forward_noalloc on the current device; code 0 =
    none of them gave up a bounded wait. ``reset`` clears the word after reading."""
    out = (C.c_int * 4)()
    _check(lib().efa_flash_attn_tc_noalloc_status(out, int(bool(reset))), "flash_attn_tc_noalloc_status")
    return tuple(out)


def flash_attn_tc_combine(part: FlashPartials, O, row0: int, rows: int, fp: FlashParams, stream=None,
                          o_dtype: int = F16) -> None:
    """flash_attn_tc_combine (flash_attn_tc.cuh:54-57)."""
    _check(lib().efa_flash_attn_tc_combine(C.byref(part), _ptr(O), o_dtype, row0, rows, C.byref(fp), _stream(stream)),
           "flash_attn_tc_combine")


def convert_f32_to_f16(src, dst, n: int, stream=None) -> None:
    _check(lib().efa_convert_f32_to_f16(_ptr(src), _ptr(dst), n, _stream(stream)), "convert_f32_to_f16")


def project(O_tile, W_O, out, rows: int, d_local: int, d: int, stream=None) -> None:
    """project (attn_main.cu:262-273) on fp16 data: out[rows][d] = O_tile[rows][d_local] @ W_O[d_local][d]."""
    _check(lib().efa_project_f16(_ptr(O_tile), _ptr(W_O), _ptr(out), rows, d_local, d, _stream(stream)), "project")


def compute_qkv(X, W_q, W_k, W_v, Qh, Kh, Vh, S: int, d: int, H_local: int, d_h: int, stream=None) -> None:
    """compute_qkv (attn_main.cu:127-153) on fp16 data: Q/K/V = X @ W per head, written fp16 head-major."""
    _check(lib().efa_compute_qkv_f16(_ptr(X), _ptr(W_q), _ptr(W_k), _ptr(W_v), _ptr(Qh), _ptr(Kh), _ptr(Vh),
                                     S, d, H_local, d_h, _stream(stream)), "compute_qkv")


def kernel_status() -> Sequence[int]:
    out = (C.c_int * 4)()
    _check(lib().efa_kernel_status(out), "kernel_status")
    return tuple(out)


def kernel_status_reset() -> None:
    _check(lib().efa_kernel_status_reset(), "kernel_status_reset")


# ------------------------------------------------------------------------------------------------
# Runtime
# ------------------------------------------------------------------------------------------------
class World:
    """Host control plane of one rank (what MPI is to the reference: barrier, max, broadcast).

    ``World()`` is a single rank. ``World.from_torch(group)`` runs the callbacks over a
    torch.distributed process group whose backend accepts CPU tensors (gloo).
    """

    def __init__(self, rank: int = 0, size: int = 1, local_device: int = 0, group=None):
        self.rank, self.size, self.local_device, self.group = rank, size, local_device, group
        self._cbs = []
        self.struct = WorldStruct()
        self.struct.user = None
        self.struct.rank, self.struct.size, self.struct.local_device = rank, size, local_device
        if size > 1:
            self._install(group)      # group None = torch.distributed's default group

    @classmethod
    def from_torch(cls, group=None, local_device: Optional[int] = None) -> "World":
        import torch.distributed as dist
        rank, size = dist.get_rank(group), dist.get_world_size(group)
        if local_device is None:
            local_device = int(os.environ.get("LOCAL_RANK", rank))
        return cls(rank, size, local_device, group) if size > 1 else cls(0, 1, local_device)

    def _install(self, group) -> None:
        import torch
        import torch.distributed as dist

        def barrier(_user):
            try:
                dist.barrier(group=group)
                return 0
            except Exception:           # reported to the C side as a failed collective
                return 1

        def allmax(_user, value):
            try:
                t = torch.tensor([value[0]], dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                value[0] = float(t[0])
                return 0
            except Exception:
                return 1

        def bcast(_user, buf, n, root):
            try:
                arr = (C.c_ubyte * n).from_address(buf)
                t = torch.frombuffer(arr, dtype=torch.uint8).clone()
                dist.broadcast(t, src=dist.get_global_rank(group, root) if group is not None else root, group=group)
                C.memmove(buf, t.numpy().ctypes.data, n)
                return 0
            except Exception:
                return 1

        def gather(_user, src, dst, n):
            try:
                arr = (C.c_ubyte * n).from_address(src)
                t = torch.frombuffer(arr, dtype=torch.uint8).clone()
                outs = [torch.empty(n, dtype=torch.uint8) for _ in range(self.size)]
                dist.all_gather(outs, t, group=group)
                for r, o in enumerate(outs):
                    C.memmove(dst + r * n, o.numpy().ctypes.data, n)
                return 0
            except Exception:
                return 1

        self._cbs = [_BARRIER_FN(barrier), _MAX_FN(allmax), _BCAST_FN(bcast), _GATHER_FN(gather)]
        self.struct.barrier, self.struct.allreduce_max_f64, self.struct.bcast_bytes, self.struct.allgather_bytes = self._cbs


def world_selftest(world: World) -> None:
    """Run every control-plane callback once and check the results (host only)."""
    _check(lib().efa_world_selftest(C.byref(world.struct)), "world_selftest")


class Ctx:
    """RunCtx (attn_defs.cuh:86-99) made by make_ctx (attn_main.cu:180-202)."""

    def __init__(self, world: World, ncomm: int = 1, prioritize: bool = True):
        self.world = world           # keeps the callbacks alive
        self.handle = C.c_void_p()
        _check(lib().efa_make_ctx(C.byref(self.handle), C.byref(world.struct), ncomm, int(prioritize)), "make_ctx")

    def destroy(self) -> None:
        if self.handle:
            lib().efa_destroy_ctx(self.handle)
            self.handle = C.c_void_p()


def make_ctx(world: World, ncomm: int = 1, prioritize: bool = True) -> Ctx:
    return Ctx(world, ncomm, prioritize)


def nvls_output(ctx: Ctx, p: Params) -> int:
    """Device address of an fp16 [S][d] output buffer inside the context's multicast region, which the NVLS reduction
    writes in place (collective). Valid until the context is destroyed or the region grows."""
    out = C.c_void_p()
    _check(lib().efa_nvls_output(ctx.handle, C.byref(p), C.byref(out)), "nvls_output")
    return int(out.value)


def set_wait_limit_ms(ctx: Ctx, device_ms: float = 0.0, host_ms: float = 0.0) -> None:
    """Limits of the guarded waits: how long a kernel polls a counter or flag that never comes before it reports
    a status, and how long run_mode waits for a stream before it releases pending counter waits (<= 0: unchanged)."""
    _check(lib().efa_ctx_set_wait_limit_ms(ctx.handle, float(device_ms), float(host_ms)), "set_wait_limit_ms")


def destroy_ctx(ctx: Ctx) -> None:
    ctx.destroy()


def fill_host_inputs(p: Params, rank: int, seed: int, recipe: int, Qh, Kh, Vh, W_O) -> None:
    """Write this rank's synthetic fp16 inputs into host arrays (numpy uint16/float16 or pinned tensors)."""
    _check(lib().efa_fill_host_inputs(C.byref(p), rank, seed, recipe, _ptr(Qh), _ptr(Kh), _ptr(Vh), _ptr(W_O)),
           "fill_host_inputs")


def run_mode(ctx: Ctx, mode: int, w: Weights, output, p: Params) -> RunStats:
    """run_mode (run_drivers.cu:277-292). ``output``: fp16 [S][d] on the device. Returns the timing record."""
    st = RunStats()
    _check(lib().efa_run_mode(ctx.handle, mode, C.byref(w), _ptr(output), C.byref(p), C.byref(st)),
           f"run_mode({MODE_NAMES[mode] if 0 <= mode < 7 else mode})")
    return st


def run_mode_residual(ctx: Ctx, mode: int, w: Weights, residual, output, p: Params) -> RunStats:
    """The block plus the step after it: ``output = residual + reduced`` with the residual (fp16 [S][d] on the
    device) added to each reduced group of rows as it lands."""
    st = RunStats()
    _check(lib().efa_run_mode_residual(ctx.handle, mode, C.byref(w), _ptr(residual), _ptr(output), C.byref(p), C.byref(st)),
           f"run_mode_residual({MODE_NAMES[mode] if 0 <= mode < 7 else mode})")
    return st


def run_mode_host(ctx: Ctx, mode: int, Qh, Kh, Vh, W_O, output, p: Params, out_row0: int = 0,
                  out_rows: Optional[int] = None) -> RunStats:
    """The block on host buffers (copies inside the timed region). ``output`` receives rows
    [out_row0, out_row0 + out_rows) of the result (all of them by default; None: nothing is copied back)."""
    st = RunStats()
    if out_rows is None:
        out_rows = p.S - out_row0 if output is not None else 0
    _check(lib().efa_run_mode_host_rows(ctx.handle, mode, _ptr(Qh), _ptr(Kh), _ptr(Vh), _ptr(W_O), _ptr(output),
                                        out_row0, out_rows, C.byref(p), C.byref(st)), "run_mode_host")
    return st
