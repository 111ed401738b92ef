"""ctypes binding of the C ABI in include/ccglib_b200.h (harness for tests and benchmarks)."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# CCGLIB_B200_LIB selects another build of the same library (e.g. an instrumented one)
LIB_PATH = os.environ.get("CCGLIB_B200_LIB") or os.path.join(HERE, "lib", "libccglib_b200.so")

# ccglib::ValueType (reference include/ccglib/common/value_type.h:14-22)
INT1, INT32, BFLOAT16, FLOAT8E4M3, FLOAT8E5M2, FLOAT16, FLOAT32 = range(7)
BASIC, OPT = 0, 1
ROW_MAJOR, COL_MAJOR = 0, 1
PLANAR, INTERLEAVED = 0, 1
FORWARD, BACKWARD = 0, 1

OK, INVALID_ARGUMENT, UNSUPPORTED, CUDA_ERROR, DEVICE_TIMEOUT, OUT_OF_MEMORY = range(6)

EXPORTS = [
    "ccglib_b200_gemm_dims", "ccglib_b200_gemm_plan_create", "ccglib_b200_gemm_run",
    "ccglib_b200_gemm_plan_destroy", "ccglib_b200_gemm_plan_scratch_bytes",
    "ccglib_b200_gemm_plan_launches", "ccglib_b200_gemm_plan_tile",
    "ccglib_b200_tune_table_lookup", "ccglib_b200_batch_share",
    "ccglib_b200_transpose_run", "ccglib_b200_pack_run", "ccglib_b200_device_status",
    "ccglib_b200_status_string", "ccglib_b200_last_error",
    "ccglib_b200_gemm_int1_static_scratch", "ccglib_b200_selftest_wait_timeout",
    "ccglib_b200_pipeline_create", "ccglib_b200_pipeline_run", "ccglib_b200_pipeline_run_host",
    "ccglib_b200_pipeline_host_slice", "ccglib_b200_pipeline_set_host_slice",
    "ccglib_b200_pipeline_launches", "ccglib_b200_pipeline_scratch_bytes",
    "ccglib_b200_pipeline_set_gemm_events", "ccglib_b200_pipeline_set_overlap",
    "ccglib_b200_pipeline_destroy",
]


class GemmDesc(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_size_t), ("m", ctypes.c_size_t), ("n", ctypes.c_size_t),
                ("k", ctypes.c_size_t), ("type_in", ctypes.c_int), ("type_out", ctypes.c_int),
                ("variant", ctypes.c_int), ("c_complex_axis", ctypes.c_int),
                ("a_mem_order", ctypes.c_int), ("b_mem_order", ctypes.c_int),
                ("c_mem_order", ctypes.c_int), ("alpha_re", ctypes.c_float),
                ("alpha_im", ctypes.c_float), ("beta_re", ctypes.c_float),
                ("beta_im", ctypes.c_float)]


class PipelineDesc(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_size_t), ("m", ctypes.c_size_t), ("n", ctypes.c_size_t),
                ("k", ctypes.c_size_t), ("type_in", ctypes.c_int), ("type_out", ctypes.c_int),
                ("variant", ctypes.c_int), ("input_complex_axis", ctypes.c_int),
                ("output_complex_axis", ctypes.c_int), ("a_mem_order", ctypes.c_int),
                ("b_mem_order", ctypes.c_int), ("c_mem_order", ctypes.c_int),
                ("alpha_re", ctypes.c_float), ("alpha_im", ctypes.c_float),
                ("beta_re", ctypes.c_float), ("beta_im", ctypes.c_float)]


class Share(ctypes.Structure):
    _fields_ = [(name, ctypes.c_size_t) for name in
                ("first", "count", "a_offset", "b_offset", "c_offset", "a_bytes", "b_bytes",
                 "c_bytes")]


class Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__("ccglib_b200 status %d (%s): %s" % (status, STATUS_NAMES.get(status, "?"),
                                                          message))
        self.status = status
        self.message = message


STATUS_NAMES = {0: "OK", 1: "INVALID_ARGUMENT", 2: "UNSUPPORTED", 3: "CUDA_ERROR",
                4: "DEVICE_TIMEOUT", 5: "OUT_OF_MEMORY"}

_lib = None


def lib() -> ctypes.CDLL:
    """Load the CUDA library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: run `python -m ccglib_b200.build` "
                              "(there is no CPU fallback)" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        L.ccglib_b200_gemm_dims.argtypes = [ci, ci, ci, ctypes.POINTER(ctypes.c_uint * 3)]
        L.ccglib_b200_gemm_dims.restype = ci
        L.ccglib_b200_gemm_plan_create.argtypes = [ctypes.POINTER(GemmDesc), ctypes.POINTER(vp)]
        L.ccglib_b200_gemm_plan_create.restype = ci
        L.ccglib_b200_gemm_run.argtypes = [vp, vp, vp, vp, vp]
        L.ccglib_b200_gemm_run.restype = ci
        L.ccglib_b200_gemm_plan_destroy.argtypes = [vp]
        L.ccglib_b200_gemm_plan_destroy.restype = ci
        L.ccglib_b200_gemm_plan_scratch_bytes.argtypes = [vp]
        L.ccglib_b200_gemm_plan_scratch_bytes.restype = sz
        L.ccglib_b200_gemm_plan_tile.argtypes = [vp, ctypes.POINTER(ci * 5)]
        L.ccglib_b200_gemm_plan_tile.restype = ci
        L.ccglib_b200_tune_table_lookup.argtypes = [ctypes.c_char_p, ctypes.POINTER(GemmDesc),
                                                    ctypes.POINTER(ci * 3)]
        L.ccglib_b200_tune_table_lookup.restype = ci
        L.ccglib_b200_batch_share.argtypes = [ctypes.POINTER(GemmDesc), ci, ci,
                                              ctypes.POINTER(Share)]
        L.ccglib_b200_batch_share.restype = ci
        L.ccglib_b200_gemm_plan_launches.argtypes = [vp]
        L.ccglib_b200_gemm_plan_launches.restype = sz
        L.ccglib_b200_gemm_int1_static_scratch.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp]
        L.ccglib_b200_gemm_int1_static_scratch.restype = ci
        L.ccglib_b200_transpose_run.argtypes = [sz, sz, sz, sz, sz, sz, ci, vp, vp, vp]
        L.ccglib_b200_transpose_run.restype = ci
        L.ccglib_b200_pack_run.argtypes = [sz, ci, ci, vp, vp, vp]
        L.ccglib_b200_pack_run.restype = ci
        L.ccglib_b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        L.ccglib_b200_device_status.restype = ci
        L.ccglib_b200_selftest_wait_timeout.argtypes = [ctypes.c_longlong, ci,
                                                        ctypes.POINTER(ctypes.c_longlong * 2)]
        L.ccglib_b200_selftest_wait_timeout.restype = ci
        L.ccglib_b200_pipeline_create.argtypes = [ctypes.POINTER(PipelineDesc), ctypes.POINTER(vp)]
        L.ccglib_b200_pipeline_create.restype = ci
        L.ccglib_b200_pipeline_run.argtypes = [vp, vp, vp, vp, vp]
        L.ccglib_b200_pipeline_run.restype = ci
        L.ccglib_b200_pipeline_run_host.argtypes = [vp, vp, vp, vp, vp]
        L.ccglib_b200_pipeline_run_host.restype = ci
        L.ccglib_b200_pipeline_host_slice.argtypes = [vp]
        L.ccglib_b200_pipeline_host_slice.restype = sz
        L.ccglib_b200_pipeline_set_host_slice.argtypes = [vp, sz]
        L.ccglib_b200_pipeline_set_host_slice.restype = ci
        L.ccglib_b200_pipeline_set_gemm_events.argtypes = [vp, vp, vp]
        L.ccglib_b200_pipeline_set_gemm_events.restype = ci
        L.ccglib_b200_pipeline_set_overlap.argtypes = [vp, ci]
        L.ccglib_b200_pipeline_set_overlap.restype = ci
        L.ccglib_b200_pipeline_launches.argtypes = [vp]
        L.ccglib_b200_pipeline_launches.restype = sz
        L.ccglib_b200_pipeline_scratch_bytes.argtypes = [vp]
        L.ccglib_b200_pipeline_scratch_bytes.restype = sz
        L.ccglib_b200_pipeline_destroy.argtypes = [vp]
        L.ccglib_b200_pipeline_destroy.restype = ci
        L.ccglib_b200_status_string.argtypes = [ci]
        L.ccglib_b200_status_string.restype = ctypes.c_char_p
        L.ccglib_b200_last_error.argtypes = []
        L.ccglib_b200_last_error.restype = ctypes.c_char_p
        _lib = L
    return _lib


def _check(status: int) -> None:
    if status != OK:
        raise Error(status, lib().ccglib_b200_last_error().decode())


def gemm_dims(type_in: int, type_out: int = FLOAT32, variant: int = OPT) -> tuple[int, int, int]:
    dims = (ctypes.c_uint * 3)()
    _check(lib().ccglib_b200_gemm_dims(type_in, type_out, variant, ctypes.byref(dims)))
    return int(dims[0]), int(dims[1]), int(dims[2])


class GemmPlan:
    """Owns a ccglib_b200_gemm_plan (the counterpart of a ccglib::mma::GEMM object)."""

    def __init__(self, batch, m, n, k, type_in, type_out, variant=OPT, c_complex_axis=PLANAR,
                 c_mem_order=ROW_MAJOR, a_mem_order=ROW_MAJOR, b_mem_order=COL_MAJOR,
                 alpha=(1.0, 0.0), beta=(0.0, 0.0)):
        self.desc = GemmDesc(batch, m, n, k, type_in, type_out, variant, c_complex_axis,
                             a_mem_order, b_mem_order, c_mem_order, alpha[0], alpha[1], beta[0],
                             beta[1])
        self._plan = ctypes.c_void_p()
        _check(lib().ccglib_b200_gemm_plan_create(ctypes.byref(self.desc),
                                                  ctypes.byref(self._plan)))

    @property
    def scratch_bytes(self) -> int:
        return int(lib().ccglib_b200_gemm_plan_scratch_bytes(self._plan))

    @property
    def launches(self) -> int:
        """Kernel launches one run() enqueues."""
        return int(lib().ccglib_b200_gemm_plan_launches(self._plan))

    @property
    def tile(self) -> dict:
        """Tile choice of the plan: columns, CTA pair, panel width from a table, tuned or not."""
        t = (ctypes.c_int * 5)()
        _check(lib().ccglib_b200_gemm_plan_tile(self._plan, ctypes.byref(t)))
        return {"bn": int(t[0]), "pair": int(t[1]), "group_n": int(t[2]), "tuned": bool(t[3]),
                "split_k": int(t[4])}

    def run(self, d_a: int, d_b: int, d_c: int, stream: int = 0) -> None:
        _check(lib().ccglib_b200_gemm_run(self._plan, d_a, d_b, d_c, stream))

    def close(self) -> None:
        if self._plan:
            lib().ccglib_b200_gemm_plan_destroy(self._plan)
            self._plan = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Pipeline:
    """Owns a ccglib_b200_pipeline (the counterpart of a ccglib::pipeline::Pipeline object)."""

    def __init__(self, batch, m, n, k, type_in, type_out, variant=OPT, input_complex_axis=PLANAR,
                 output_complex_axis=PLANAR, c_mem_order=ROW_MAJOR, a_mem_order=ROW_MAJOR,
                 b_mem_order=COL_MAJOR, alpha=(1.0, 0.0), beta=(0.0, 0.0)):
        self.desc = PipelineDesc(batch, m, n, k, type_in, type_out, variant, input_complex_axis,
                                 output_complex_axis, a_mem_order, b_mem_order, c_mem_order,
                                 alpha[0], alpha[1], beta[0], beta[1])
        self._p = ctypes.c_void_p()
        _check(lib().ccglib_b200_pipeline_create(ctypes.byref(self.desc), ctypes.byref(self._p)))

    @property
    def launches(self) -> int:
        return int(lib().ccglib_b200_pipeline_launches(self._p))

    @property
    def scratch_bytes(self) -> int:
        return int(lib().ccglib_b200_pipeline_scratch_bytes(self._p))

    @property
    def host_slice(self) -> int:
        return int(lib().ccglib_b200_pipeline_host_slice(self._p))

    @host_slice.setter
    def host_slice(self, items: int) -> None:
        _check(lib().ccglib_b200_pipeline_set_host_slice(self._p, items))

    def set_overlap(self, on: bool) -> None:
        """Transposes of later batch chunks beside the GEMM of earlier ones (default) or the
        plain chain on the caller's stream."""
        _check(lib().ccglib_b200_pipeline_set_overlap(self._p, 1 if on else 0))

    def set_gemm_events(self, begin: int | None, end: int | None) -> None:
        """CUDA event handles recorded around the GEMM stage of every later run (None: off)."""
        _check(lib().ccglib_b200_pipeline_set_gemm_events(self._p, begin, end))

    def run(self, d_a: int, d_b: int, d_c: int, stream: int = 0) -> None:
        _check(lib().ccglib_b200_pipeline_run(self._p, d_a, d_b, d_c, stream))

    def run_host(self, h_a: int, h_b: int, h_c: int, stream: int = 0) -> None:
        """Host pointers of the whole A, B, C; returns when C is complete."""
        _check(lib().ccglib_b200_pipeline_run_host(self._p, h_a, h_b, h_c, stream))

    def close(self) -> None:
        if self._p:
            lib().ccglib_b200_pipeline_destroy(self._p)
            self._p = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def batch_share(batch, m, n, k, type_in, type_out, variant, world, rank) -> dict:
    """Rank's contiguous share of a batch split over `world` devices (host arithmetic)."""
    desc = GemmDesc(batch, m, n, k, type_in, type_out, variant, PLANAR, ROW_MAJOR, COL_MAJOR,
                    ROW_MAJOR, 1.0, 0.0, 0.0, 0.0)
    share = Share()
    _check(lib().ccglib_b200_batch_share(ctypes.byref(desc), world, rank, ctypes.byref(share)))
    keys = {"first": "first", "count": "count", "a": "a_offset", "b": "b_offset",
            "c": "c_offset", "a_bytes": "a_bytes", "b_bytes": "b_bytes", "c_bytes": "c_bytes"}
    return {k: int(getattr(share, v)) for k, v in keys.items()}


def tune_table_lookup(path: str, batch, m, n, k, type_in, type_out):
    """(bn, pair, group_n) a tuning table file holds for a problem, or None (host only)."""
    desc = GemmDesc(batch, m, n, k, type_in, type_out, OPT, PLANAR, ROW_MAJOR, COL_MAJOR,
                    ROW_MAJOR, 1.0, 0.0, 0.0, 0.0)
    choice = (ctypes.c_int * 3)()
    status = lib().ccglib_b200_tune_table_lookup(path.encode(), ctypes.byref(desc),
                                                 ctypes.byref(choice))
    if status == UNSUPPORTED:
        return None
    _check(status)
    return int(choice[0]), int(choice[1]), int(choice[2])


def gemm_int1_static_scratch(batch, m, n, k, d_a, d_b, d_c, stream: int = 0, variant=BASIC,
                             c_complex_axis=PLANAR, c_mem_order=ROW_MAJOR, alpha=(1.0, 0.0),
                             beta=(0.0, 0.0)) -> None:
    """1-bit GEMM through the entry point that takes its scratch from the library's built-in
    array instead of allocating (see include/ccglib_b200.h)."""
    desc = GemmDesc(batch, m, n, k, INT1, INT32, variant, c_complex_axis, ROW_MAJOR, COL_MAJOR,
                    c_mem_order, alpha[0], alpha[1], beta[0], beta[1])
    _check(lib().ccglib_b200_gemm_int1_static_scratch(ctypes.byref(desc), d_a, d_b, d_c, stream))


def transpose(batch, m, n, m_chunk, n_chunk, nr_bits, input_complex_axis, d_in, d_out,
              stream: int = 0) -> None:
    _check(lib().ccglib_b200_transpose_run(batch, m, n, m_chunk, n_chunk, nr_bits,
                                           input_complex_axis, d_in, d_out, stream))


def pack(n, direction, input_complex_axis, d_in, d_out, stream: int = 0) -> None:
    _check(lib().ccglib_b200_pack_run(n, direction, input_complex_axis, d_in, d_out, stream))


def selftest_wait_timeout(limit_cycles: int, pair: bool = False) -> tuple[int, int]:
    """Make a bounded device-side wait run out (see include/ccglib_b200.h); returns the cycles
    the two waiters spent.  The device status word is left set."""
    waited = (ctypes.c_longlong * 2)()
    _check(lib().ccglib_b200_selftest_wait_timeout(limit_cycles, 1 if pair else 0,
                                                   ctypes.byref(waited)))
    return int(waited[0]), int(waited[1])


def device_status() -> int:
    """Synchronise, then read and clear the device status word (0 = no device-side time-out)."""
    word = ctypes.c_uint(0)
    status = lib().ccglib_b200_device_status(ctypes.byref(word))
    if status not in (OK, DEVICE_TIMEOUT):
        _check(status)
    return int(word.value)
