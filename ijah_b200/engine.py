"""ctypes binding of libijah_b200.so: the host-side mirror of the reference's tools/engine.py (same class and method
names for the part of the C ABI this library implements: Engine, Buf, Pack, FnLayer) plus the dimension-explicit
operators of include/ijah_b200.h (Exl3Linear, MoeBlock).

    from ijah_b200 import engine as E
    eng = E.Engine()                       # loads ijah_b200/libijah_b200.so (NE_LIB overrides, as in the reference)
    p = eng.pack_open(pack_dir)
    L = eng.fn_layer(p, 0, rows=4)         # MoE block of layer 0
    L.write("mlp_in", x); L.run_stage(5); y = L.read("mlp_out")

There is no fallback: if the shared library is missing or a call fails, EngineError is raised. Device memory for the
operator classes is held in torch CUDA tensors (torch is plumbing here: allocation, streams, torch.distributed).
"""
import ctypes as C
import json
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = Path(os.environ.get("NE_LIB", HERE / "libijah_b200.so"))
MAX_DIMS = 8
DTYPES = {0: "F32", 1: "F16", 2: "BF16", 3: "U8", 4: "U16", 5: "U32", 6: "I32", 7: "I64", 8: "I8", 9: "I16",
          10: "U64", 11: "F64", 12: "BOOL"}
NP = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "U8": np.uint8, "U16": np.uint16, "U32": np.uint32,
      "I32": np.int32, "I64": np.int64, "I8": np.int8, "I16": np.int16, "U64": np.uint64, "F64": np.float64,
      "BOOL": np.uint8}


class DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("has_nax", C.c_int), ("has_metal4", C.c_int),
                ("max_buffer_length", C.c_uint64), ("recommended_working_set", C.c_uint64),
                ("max_threadgroup_memory", C.c_uint64), ("backend", C.c_char * 16)]


class TensorDescC(C.Structure):
    _fields_ = [("dtype", C.c_int), ("ndim", C.c_int), ("shape", C.c_int64 * MAX_DIMS), ("nbytes", C.c_uint64),
                ("file", C.c_char_p), ("file_offset", C.c_uint64), ("host", C.c_void_p), ("buf", C.c_void_p),
                ("buf_offset", C.c_uint64)]


class Exl3WeightC(C.Structure):
    _fields_ = [("trellis", C.c_void_p), ("suh", C.c_void_p), ("svh", C.c_void_p), ("n_in", C.c_int),
                ("n_out", C.c_int), ("K", C.c_int)]


class Q8WeightC(C.Structure):  # include/ijah_b200.h: ne_q8_weight
    _fields_ = [("weight", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p), ("n_in", C.c_int), ("n_out", C.c_int),
                ("group", C.c_int)]


class Exl3StackC(C.Structure):
    _fields_ = [("trellis", C.c_void_p), ("suh", C.c_void_p), ("svh", C.c_void_p)]


class MoeDescC(C.Structure):
    _fields_ = [("hidden", C.c_int), ("inter", C.c_int), ("experts", C.c_int), ("top_k", C.c_int),
                ("k_expert", C.c_int), ("k_shared", C.c_int), ("expert_first", C.c_int), ("expert_count", C.c_int),
                ("router", C.c_void_p), ("shared_gate_w", C.c_void_p), ("gate", Exl3StackC), ("up", Exl3StackC),
                ("down", Exl3StackC), ("sh_gate", Exl3WeightC), ("sh_up", Exl3WeightC), ("sh_down", Exl3WeightC),
                ("sh_gate_q8", Q8WeightC), ("sh_up_q8", Q8WeightC), ("sh_down_q8", Q8WeightC)]


class ModelDescC(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("layers", "hidden", "inter", "experts", "top_k", "k_expert", "k_shared", "q_out", "kv_out",
                                       "heads", "kv_heads", "head_dim", "k_trunk", "k_trunk_alt", "alt_every", "vocab",
                                       "kv_positions", "expert_first", "expert_count", "ep_world")]


class ArgC(C.Structure):  # ne_arg: a buffer with a byte offset, or inline bytes
    _fields_ = [("buf", C.c_void_p), ("offset", C.c_uint64), ("bytes", C.c_void_p), ("nbytes", C.c_uint32)]


class EngineError(RuntimeError):
    pass


# every symbol include/ijah_engine.h and include/ijah_b200.h declare: (restype, argtypes)
SIGNATURES = {
    "ne_abi_version": (C.c_int, []), "ne_last_error": (C.c_char_p, []),
    "ne_dtype_name": (C.c_char_p, [C.c_int]), "ne_dtype_size": (C.c_int, [C.c_int]),
    "ne_device_query": (C.c_int, [C.POINTER(DeviceInfo)]),
    "ne_alloc": (C.c_void_p, [C.c_uint64]), "ne_free": (None, [C.c_void_p]),
    "ne_buf_size": (C.c_uint64, [C.c_void_p]), "ne_buf_contents": (C.c_void_p, [C.c_void_p]),
    "ne_buf_gpu_address": (C.c_uint64, [C.c_void_p]),
    "ne_upload": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "ne_download": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "ne_pack_open": (C.c_void_p, [C.c_char_p]), "ne_pack_close": (None, [C.c_void_p]),
    "ne_pack_config_json": (C.c_char_p, [C.c_void_p]), "ne_pack_num_tensors": (C.c_int64, [C.c_void_p]),
    "ne_pack_tensor_name": (C.c_char_p, [C.c_void_p, C.c_int64]),
    "ne_tensor_info": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(TensorDescC)]),
    "ne_pack_view_rows": (C.c_void_p, [C.c_void_p, C.c_char_p, C.c_int64, C.c_int64, C.POINTER(C.c_uint64)]),
    "ne_kernel_exists": (C.c_int, [C.c_char_p]),
    "ne_run_kernel": (C.c_int, [C.c_char_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                C.c_uint32, C.c_int, C.c_char_p, C.POINTER(C.c_double)]),
    "ne_fn_layer_create": (C.c_void_p, [C.c_void_p, C.c_int]),
    "ne_fn_layer_create_rows": (C.c_void_p, [C.c_void_p, C.c_int, C.c_int]),
    "ne_fn_layer_free": (None, [C.c_void_p]),
    "ne_fn_layer_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_double)]),
    "ne_fn_layer_run_stage": (C.c_int, [C.c_void_p, C.c_int]),
    "ne_fn_layer_run_dispatch": (C.c_int, [C.c_void_p, C.c_int]),
    "ne_fn_set_ref_rounding": (C.c_int, [C.c_int]),
    "ne_fn_layer_write": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int]),
    "ne_fn_layer_read": (C.c_int, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int]),
    "ne_fn_layer_time": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "ne_exl3_dequant": (C.c_int, [C.POINTER(Exl3WeightC), C.c_void_p, C.c_void_p]),
    "ne_exl3_linear": (C.c_int, [C.POINTER(Exl3WeightC), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_q8_linear": (C.c_int, [C.POINTER(Q8WeightC), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_q8_embed": (C.c_int, [C.POINTER(Q8WeightC), C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "ne_exl3_linear_host": (C.c_int, [C.POINTER(Exl3WeightC), C.c_void_p, C.c_int, C.c_void_p]),
    "ne_exl3_linear_plan": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_uint64)]),
    "ne_moe_plan": (C.c_int, [C.c_int] * 7 + [C.POINTER(C.c_int)]),
    "ne_exl3_linear_multi": (C.c_int, [C.POINTER(Exl3WeightC), C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.c_void_p]),
    "ne_exl3_linear_prefill": (C.c_int, [C.POINTER(Exl3WeightC), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_exl3_linear_static": (C.c_int, [C.POINTER(Exl3WeightC), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_exl3_linear_static_capacity": (C.c_uint64, []),
    "ne_moe_create": (C.c_void_p, [C.POINTER(MoeDescC), C.c_int]), "ne_moe_free": (None, [C.c_void_p]),
    "ne_moe_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_moe_forward_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "ne_moe_stage": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_moe_forward_routed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_moe_prefill": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_moe_route": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "ne_moe_forward_ep_routed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                           C.c_void_p]),
    "ne_ep_create": (C.c_void_p, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "ne_ep_handle": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ne_ep_connect": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ne_ep_free": (None, [C.c_void_p]), "ne_ep_disconnect": (C.c_int, [C.c_void_p]),
    "ne_moe_forward_ep_fused": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_moe_prefill_ep": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_moe_forward_ep": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_moe_prefill_home": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ne_moe_prefill_routed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_ep_pairs_by_owner": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ne_rows_gather": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "ne_slots_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "ne_moe_buffer": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]),
    "ne_moe_experts_gu": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "ne_moe_last_bytes": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64),
                                    C.POINTER(C.c_uint64), C.POINTER(C.c_int)]),
    "ne_fn_model_create": (C.c_void_p, [C.c_void_p, C.c_int]),
    "ne_fn_model_create_rows": (C.c_void_p, [C.c_void_p, C.c_int, C.c_int]),
    "ne_fn_model_create_synthetic": (C.c_void_p, [C.POINTER(ModelDescC), C.c_uint64, C.c_int]),
    "ne_fn_model_free": (None, [C.c_void_p]), "ne_fn_model_reset": (C.c_int, [C.c_void_p]),
    "ne_fn_model_step": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_float),
                                   C.POINTER(C.c_int), C.POINTER(C.c_double)]),
    "ne_fn_model_step_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.POINTER(C.c_double)]),
    "ne_fn_model_time": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "ne_fn_model_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "ne_fn_model_prefill": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_double)]),
    "ne_fn_model_verify_greedy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_int), C.c_void_p, C.POINTER(C.c_double)]),
    "ne_fn_model_replay": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double)]),
    "ne_fn_model_desc_of": (C.c_int, [C.c_void_p, C.POINTER(ModelDescC)]),
    "ne_fn_model_set_ep": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ne_fn_model_read": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int, C.c_void_p, C.c_uint64]),
    "ne_fn_model_weight_bytes": (C.c_uint64, [C.c_void_p]),
    "ne_fn_model_last_bytes": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_int)]),
    "ne_copy_to_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64]),
    "ne_device_wait_status": (C.c_int, []),
    "ne_exl3_set_summand_product": (C.c_int, [C.c_int]),
}


def load_library(path=None):
    path = Path(path or LIB)
    if not path.exists():
        raise EngineError(f"{path} is not built (run `make -C ijah_b200/csrc` or __graft_entry__.build())")
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        f = getattr(lib, name)  # AttributeError if a declared symbol is not exported
        f.restype, f.argtypes = res, args
    return lib


class _Owned:
    """Base of the wrappers around an opaque C handle: remembers the engine, releases the handle once (explicitly with
    free() / close(), or when used as a context manager) and refuses further use afterwards."""

    _release = None  # name of the C function that releases the handle

    def __init__(self, eng, ptr, what):
        if not ptr:
            raise EngineError(f"{what}: {eng.last_error()}")
        self.eng, self.ptr = eng, ptr

    def _live(self):
        if not self.ptr:
            raise EngineError(f"{type(self).__name__} used after it was released")
        return self.ptr

    def free(self):
        ptr, self.ptr = self.ptr, None
        if ptr and self._release:
            getattr(self.eng.lib, self._release)(ptr)

    close = free

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.free()


def _flat_count(nbytes, dtype, shape):
    return int(np.prod(shape)) if shape is not None else nbytes // np.dtype(dtype).itemsize


class Buf(_Owned):
    """A device buffer of the library (ne_buf): a managed allocation made by Engine.alloc, a device copy of pack rows, or
    -- with owned=False -- the handle of a pack tensor, which the pack releases, never this object."""

    def __init__(self, eng, ptr, owned=True):
        super().__init__(eng, ptr, "ne_buf")
        self._release = "ne_free" if owned else None
        self.owned = owned

    @property
    def size(self):
        return int(self.eng.lib.ne_buf_size(self._live()))

    def contents(self):
        """address of the bytes as the CPU sees them"""
        return self.eng.lib.ne_buf_contents(self._live())

    def gpu_address(self):
        """address of the bytes as kernels see them (a pack tensor becomes resident on the device here)"""
        addr = self.eng.lib.ne_buf_gpu_address(self._live())
        if not addr:
            raise EngineError(self.eng.last_error())
        return addr

    def upload(self, arr, offset=0):
        src = np.ascontiguousarray(arr)
        self.eng._ok(self.eng.lib.ne_upload(self._live(), int(offset), src.ctypes.data, src.nbytes), "ne_upload")

    def download(self, dtype=np.float32, shape=None, offset=0):
        out = np.empty(_flat_count(self.size - offset, dtype, shape), dtype)
        self.eng._ok(self.eng.lib.ne_download(self._live(), int(offset), out.ctypes.data, out.nbytes), "ne_download")
        return out if shape is None else out.reshape(shape)

    def numpy(self, dtype=np.float32, shape=None, offset=0):
        """the same bytes as a numpy array without a copy (managed memory: synchronise with the GPU before touching it)"""
        n = _flat_count(self.size - offset, dtype, shape)
        mem = (C.c_char * (n * np.dtype(dtype).itemsize)).from_address(self.contents() + offset)
        out = np.frombuffer(mem, dtype, n)
        return out if shape is None else out.reshape(shape)


class TensorDesc:
    """What ne_tensor_info reports about one pack tensor."""

    def __init__(self, eng, name, d):
        self.name, self.nbytes = name, int(d.nbytes)
        self.dtype = DTYPES.get(d.dtype, f"dtype{d.dtype}")
        self.shape = tuple(int(d.shape[i]) for i in range(d.ndim))
        self.file = d.file.decode() if d.file else None
        self.file_offset = int(d.file_offset)
        self.host_ptr = d.host
        self.buf = Buf(eng, d.buf, owned=False) if d.buf else None
        self.buf_offset = int(d.buf_offset)

    def host(self):
        """the tensor's bytes in the read-only file mapping as a numpy array (bf16 as uint16); valid while the pack is open"""
        elem = np.dtype(NP[self.dtype])
        mem = (C.c_char * self.nbytes).from_address(self.host_ptr)
        return np.frombuffer(mem, elem, self.nbytes // elem.itemsize).reshape(self.shape)

    def __repr__(self):
        return f"<{self.name}: {self.dtype} {list(self.shape)}>"


class Pack(_Owned):
    """An open pack directory (safetensors shards, their index, config.json)."""

    _release = "ne_pack_close"

    def __init__(self, eng, path):
        self.path = str(Path(path).expanduser())
        super().__init__(eng, eng.lib.ne_pack_open(self.path.encode()), f"ne_pack_open({self.path})")

    def config(self):
        return json.loads(self.eng.lib.ne_pack_config_json(self._live()).decode())

    def names(self):
        lib, ptr = self.eng.lib, self._live()
        return [lib.ne_pack_tensor_name(ptr, i).decode() for i in range(lib.ne_pack_num_tensors(ptr))]

    def info(self, name):
        raw = TensorDescC()
        if self.eng.lib.ne_tensor_info(self._live(), name.encode(), C.byref(raw)):
            raise KeyError(f"{name}: {self.eng.last_error()}")
        return TensorDesc(self.eng, name, raw)

    def view_rows(self, name, row0, nrows):
        """(Buf, offset): a device copy of rows [row0, row0 + nrows) of a tensor's first dimension, owned by the caller"""
        offset = C.c_uint64(0)
        ptr = self.eng.lib.ne_pack_view_rows(self._live(), name.encode(), row0, nrows, C.byref(offset))
        return Buf(self.eng, ptr), int(offset.value)


class FnLayer(_Owned):
    """The MoE block of one decoder layer behind the reference's layer entry points; every named buffer crosses the ABI as
    float32 host memory."""

    _release = "ne_fn_layer_free"

    def __init__(self, eng, pack, layer, rows=1):
        super().__init__(eng, eng.lib.ne_fn_layer_create_rows(pack.ptr, layer, rows), f"ne_fn_layer_create_rows(layer {layer}, {rows} rows)")
        self.layer, self.rows = layer, rows

    def _call(self, fn, *args):
        self.eng._ok(getattr(self.eng.lib, fn)(self._live(), *args), fn)

    def step(self, h_in=None):
        self._call("ne_fn_layer_step", None, None, C.byref(C.c_double(0)))  # always an error here: only the MoE block exists

    def run_stage(self, stage):
        self._call("ne_fn_layer_run_stage", int(stage))

    def run_dispatch(self, stage):
        self._call("ne_fn_layer_run_dispatch", int(stage))

    def size(self, name):
        count = self.eng.lib.ne_fn_layer_read(self._live(), name.encode(), None, 0)
        if count < 0:
            raise KeyError(f"{name}: {self.eng.last_error()}")
        return count

    def read(self, name):
        out = np.empty(self.size(name), np.float32)
        if self.eng.lib.ne_fn_layer_read(self._live(), name.encode(), out.ctypes.data, out.size) < 0:
            raise EngineError(self.eng.last_error())
        return out

    def write(self, name, arr):
        src = np.ascontiguousarray(arr, np.float32).ravel()
        self._call("ne_fn_layer_write", name.encode(), src.ctypes.data, src.size)

    def time(self, reps1=8, reps2=40, flush_mb=0):
        """(microseconds per MoE block, microseconds of the cache flush between blocks), differential over two chain lengths"""
        step_us, flush_us = C.c_double(0), C.c_double(0)
        self._call("ne_fn_layer_time", reps1, reps2, flush_mb, C.byref(step_us), C.byref(flush_us))
        return step_us.value, flush_us.value


class FnModel:
    """The decoder stack behind ne_fn_model_*: numpy in, numpy out (tokens and results cross the C ABI as host memory).
    Made from an open pack (`pack`) or, with `desc` (a dict of ne_fn_model_desc fields), from synthetic weights the
    library generates on the device."""

    def __init__(self, eng, pack=None, tmax=64, max_rows=8, desc=None, seed=1):
        self.eng = eng
        if desc is not None:
            d = ModelDescC(**desc)
            self.ptr = eng.lib.ne_fn_model_create_synthetic(C.byref(d), seed, max_rows)
        else:
            self.ptr = eng.lib.ne_fn_model_create_rows(pack.ptr, tmax, max_rows)
        if not self.ptr:
            raise EngineError(f"ne_fn_model_create: {eng.last_error()}")
        d = ModelDescC()
        eng._ok(eng.lib.ne_fn_model_desc_of(self.ptr, C.byref(d)), "ne_fn_model_desc_of")
        self.desc = {n: getattr(d, n) for n, _ in ModelDescC._fields_}
        self.max_rows = max_rows

    def step(self, token, head=True):
        """the reference's one-token step: (logits f32 [vocab], next, logprob, gpu_ms)"""
        lg = np.empty(self.desc["vocab"], np.float32)
        nx, lp, ms = C.c_int(0), C.c_float(0), C.c_double(0)
        self.eng._ok(self.eng.lib.ne_fn_model_step(self.ptr, int(token), int(head), lg.ctypes.data, C.byref(nx), C.byref(lp), None,
                                                   C.byref(ms)), "ne_fn_model_step")
        return lg, nx.value, lp.value, ms.value

    def step_rows(self, tokens, head=True, want_logits=False):
        """one decode step for len(tokens) rows: (next ids int32 [rows], logits f32 [rows, vocab] or None, gpu_ms)"""
        t = np.ascontiguousarray(tokens, np.int32)
        rows = t.shape[0]
        nx = np.zeros(rows, np.int32)
        lg = np.empty((rows, self.desc["vocab"]), np.float32) if want_logits else None
        ms = C.c_double(0)
        self.eng._ok(self.eng.lib.ne_fn_model_step_rows(self.ptr, t.ctypes.data, rows, int(head), lg.ctypes.data if want_logits else None,
                                                        nx.ctypes.data, C.byref(ms)), "ne_fn_model_step_rows")
        return nx, lg, ms.value

    def prefill(self, prompt, want_logits=True):
        """the prompt in chunks of up to max_rows rows: (greedy next token, logits of the last token or None, wall ms)"""
        ids = np.ascontiguousarray(prompt, np.int32)
        lg = np.empty(self.desc["vocab"], np.float32) if want_logits else None
        nx, ms = C.c_int(-1), C.c_double(0)
        self.eng._ok(self.eng.lib.ne_fn_model_prefill(self.ptr, ids.ctypes.data, len(ids), lg.ctypes.data if want_logits else None,
                                                      C.byref(nx), C.byref(ms)), "ne_fn_model_prefill")
        return nx.value, lg, ms.value

    def verify_greedy(self, tokens):
        """one speculative round: tokens = [last emitted, drafts...]; returns (accepted count, emitted tokens, GPU ms)"""
        ids = np.ascontiguousarray(tokens, np.int32)
        out = np.empty(len(ids), np.int32)
        acc, ms = C.c_int(0), C.c_double(0)
        self.eng._ok(self.eng.lib.ne_fn_model_verify_greedy(self.ptr, ids.ctypes.data, len(ids), C.byref(acc), out.ctypes.data, C.byref(ms)),
                     "ne_fn_model_verify_greedy")
        return acc.value, out[:acc.value + 1].copy(), ms.value

    def replay(self, rows, steps, head=True):
        """device time in ms of `steps` replays of the captured step (inputs and results stay on the device)"""
        ms = C.c_double(0)
        self.eng._ok(self.eng.lib.ne_fn_model_replay(self.ptr, rows, int(head), steps, C.byref(ms)), "ne_fn_model_replay")
        return ms.value

    def time(self, reps=10):
        a, b, c = C.c_double(0), C.c_double(0), C.c_double(0)
        self.eng._ok(self.eng.lib.ne_fn_model_time(self.ptr, 0, reps, C.byref(a), C.byref(b), C.byref(c)), "ne_fn_model_time")
        return a.value, b.value, c.value

    def info(self):
        a, b, t = C.c_int(0), C.c_int(0), C.c_int(0)
        self.eng._ok(self.eng.lib.ne_fn_model_info(self.ptr, C.byref(a), C.byref(b), C.byref(t)), "ne_fn_model_info")
        return dict(launches_full=a.value, launches_body=b.value, T=t.value)

    def read(self, name, layer=0, dtype=np.float32, count=None):
        if name in ("kv_k", "kv_v"):
            dtype, count = np.float16, self.desc["kv_positions"] * self.desc["kv_out"]
        out = np.empty(count, dtype)
        self.eng._ok(self.eng.lib.ne_fn_model_read(self.ptr, name.encode(), layer, out.ctypes.data, out.nbytes), f"ne_fn_model_read({name})")
        return out

    def set_ep(self, xchg):
        self.eng._ok(self.eng.lib.ne_fn_model_set_ep(self.ptr, xchg.ptr if xchg is not None else None), "ne_fn_model_set_ep")

    def weight_bytes(self):
        return self.eng.lib.ne_fn_model_weight_bytes(self.ptr)

    def last_bytes(self, rows):
        t, n = C.c_uint64(0), C.c_int(0)
        self.eng._ok(self.eng.lib.ne_fn_model_last_bytes(self.ptr, rows, C.byref(t), C.byref(n)), "ne_fn_model_last_bytes")
        return dict(total=t.value, distinct_experts_mean=n.value)

    def free(self):
        ptr, self.ptr = self.ptr, None
        if ptr:
            self.eng.lib.ne_fn_model_free(ptr)


class Engine:
    """The loaded library plus the factories of the handle wrappers above."""

    def __init__(self, lib=None):
        self.lib = load_library(lib)

    def last_error(self):
        msg = self.lib.ne_last_error()
        return msg.decode() if msg else ""

    def _ok(self, rc, what):
        if rc:
            raise EngineError(f"{what}: {self.last_error()}")

    def abi_version(self):
        return self.lib.ne_abi_version()

    def device(self):
        info = DeviceInfo()
        self._ok(self.lib.ne_device_query(C.byref(info)), "ne_device_query")
        text = {"name", "backend"}
        return {f: (getattr(info, f).decode() if f in text else getattr(info, f)) for f, _ in DeviceInfo._fields_}

    def alloc(self, nbytes):
        return Buf(self, self.lib.ne_alloc(int(nbytes)))

    def from_numpy(self, arr):
        src = np.ascontiguousarray(arr)
        buf = self.alloc(max(src.nbytes, 1))
        buf.upload(src)
        return buf

    def pack_open(self, path):
        return Pack(self, path)

    def fn_layer(self, pack, layer, rows=1):
        return FnLayer(self, pack, layer, rows)

    def fn_model(self, pack=None, tmax=64, max_rows=8, desc=None, seed=1):
        return FnModel(self, pack, tmax, max_rows, desc, seed)

    def kernel_exists(self, name):
        return self.lib.ne_kernel_exists(name.encode()) == 1

    def run_kernel(self, name, args, reps=1):
        """Run an operator by name (ne_run_kernel: "exl3_linear", "exl3_dequant") `reps` times; returns the GPU milliseconds of
        all repetitions. Each argument is a Buf, a (Buf, byte offset) pair, a TensorDesc of a pack tensor, or anything numpy
        can turn into bytes (passed inline)."""
        packed, keep = (ArgC * max(len(args), 1))(), []
        for slot, a in zip(packed, args):
            if isinstance(a, TensorDesc):
                a = (a.buf, a.buf_offset)
            if isinstance(a, Buf):
                a = (a, 0)
            if isinstance(a, tuple):
                slot.buf, slot.offset = a[0].ptr, int(a[1])
            else:
                blob = np.ascontiguousarray(a).tobytes()
                keep.append(C.create_string_buffer(blob, len(blob)))
                slot.bytes, slot.nbytes = C.cast(keep[-1], C.c_void_p), len(blob)
        ms = C.c_double(0)
        three = (C.c_uint32 * 3)(1, 1, 1)
        self._ok(self.lib.ne_run_kernel(name.encode(), None, 0, packed, len(args), three, three, 0, int(reps), None, C.byref(ms)),
                 f"ne_run_kernel({name})")
        return ms.value


# ------------------------------------------------------------------ dimension-explicit operators (torch for memory)
def _torch():
    import torch
    return torch


def _dev(t):
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(_torch().cuda.current_stream().cuda_stream)


def to_device_u16(a, device="cuda"):
    """numpy uint16 / float16 array (or a torch tensor already on the device) -> torch tensor of the same bits"""
    torch = _torch()
    if isinstance(a, torch.Tensor):
        return a.to(device).contiguous()
    a = np.ascontiguousarray(a)
    if a.dtype == np.float16:
        return torch.from_numpy(a).to(device)
    return torch.from_numpy(a.view(np.int16)).to(device)


class Q8Linear:
    """One 8-bit affine Linear (MLX layout) on the device: y = x @ W^T through ne_q8_linear; embedding lookup through
    ne_q8_embed. weight: uint32 [out, in / 4] (or uint8 [out, in]), scales / biases: bf16 bit patterns uint16 [out, in / group]"""

    def __init__(self, eng, weight, scales, biases, device="cuda"):
        torch = _torch()
        self.eng = eng
        w = np.ascontiguousarray(weight).view(np.uint8)
        sc, bi = np.ascontiguousarray(scales, np.uint16), np.ascontiguousarray(biases, np.uint16)
        self.n_out, self.n_in = w.shape
        self.group = self.n_in // sc.shape[1]
        self.t = (torch.from_numpy(w).to(device), to_device_u16(sc, device), to_device_u16(bi, device))
        self.c = Q8WeightC(self.t[0].data_ptr(), self.t[1].data_ptr(), self.t[2].data_ptr(), self.n_in, self.n_out, self.group)

    def __call__(self, x):
        torch = _torch()
        x = x.to(torch.float32).contiguous()
        y = torch.empty((x.shape[0], self.n_out), dtype=torch.float32, device=x.device)
        self.eng._ok(self.eng.lib.ne_q8_linear(C.byref(self.c), _dev(x), x.shape[0], _dev(y), _stream()), "ne_q8_linear")
        return y

    def embed(self, tokens, round_bf16=True):
        torch = _torch()
        t = tokens.to(torch.int32).contiguous()
        x = torch.empty((t.shape[0], self.n_in), dtype=torch.float32, device=t.device)
        self.eng._ok(self.eng.lib.ne_q8_embed(C.byref(self.c), _dev(t), t.shape[0], _dev(x), int(round_bf16), _stream()), "ne_q8_embed")
        return x


class Exl3Linear:
    """One EXL3 Linear on the device: y = x @ W through ne_exl3_linear / ne_exl3_dequant"""

    def __init__(self, eng, trellis, suh, svh, device="cuda"):
        self.eng = eng
        tr = np.asarray(trellis)
        assert tr.ndim == 3 and tr.dtype == np.uint16
        self.n_in, self.n_out, self.K = tr.shape[0] * 16, tr.shape[1] * 16, tr.shape[2] // 16
        self.t = (to_device_u16(tr, device), to_device_u16(np.asarray(suh, np.float16), device),
                  to_device_u16(np.asarray(svh, np.float16), device))
        self.c = Exl3WeightC(self.t[0].data_ptr(), self.t[1].data_ptr(), self.t[2].data_ptr(), self.n_in, self.n_out, self.K)

    @classmethod
    def from_device(cls, eng, trellis, suh, svh):
        """the same from tensors that already live on the device (int16 / uint16 trellis words, float16 scale vectors)"""
        self = cls.__new__(cls)
        self.eng = eng
        self.n_in, self.n_out, self.K = trellis.shape[0] * 16, trellis.shape[1] * 16, trellis.shape[2] // 16
        self.t = (trellis, suh, svh)
        self.c = Exl3WeightC(trellis.data_ptr(), suh.data_ptr(), svh.data_ptr(), self.n_in, self.n_out, self.K)
        return self

    def into(self, x, y):
        """y = x @ W for float32 device tensors the caller owns (no allocation, capturable)"""
        self.eng._ok(self.eng.lib.ne_exl3_linear(C.byref(self.c), _dev(x), x.shape[0], _dev(y), _stream()), "ne_exl3_linear")
        return y

    def dequant(self):
        torch = _torch()
        w = torch.empty((self.n_in, self.n_out), dtype=torch.float16, device=self.t[0].device)
        self.eng._ok(self.eng.lib.ne_exl3_dequant(C.byref(self.c), _dev(w), _stream()), "ne_exl3_dequant")
        return w

    def __call__(self, x):
        torch = _torch()
        x = x.to(torch.float32).contiguous()
        rows = x.shape[0]
        y = torch.empty((rows, self.n_out), dtype=torch.float32, device=x.device)
        self.eng._ok(self.eng.lib.ne_exl3_linear(C.byref(self.c), _dev(x), rows, _dev(y), _stream()), "ne_exl3_linear")
        return y

    def prefill(self, x):
        """many rows at once through the grouped tensor-core GEMM (ne_exl3_linear_prefill)"""
        torch = _torch()
        x = x.to(torch.float32).contiguous()
        rows = x.shape[0]
        y = torch.empty((rows, self.n_out), dtype=torch.float32, device=x.device)
        self.eng._ok(self.eng.lib.ne_exl3_linear_prefill(C.byref(self.c), _dev(x), rows, _dev(y), _stream()), "ne_exl3_linear_prefill")
        return y

    def forward_static(self, x):
        """the same Linear through ne_exl3_linear_static: scratch is the library's built-in device array, so the call
        allocates nothing in the library (the output tensor below is the caller's, made by torch)"""
        torch = _torch()
        x = x.to(torch.float32).contiguous()
        rows = x.shape[0]
        y = torch.empty((rows, self.n_out), dtype=torch.float32, device=x.device)
        self.eng._ok(self.eng.lib.ne_exl3_linear_static(C.byref(self.c), _dev(x), rows, _dev(y), _stream()),
                     "ne_exl3_linear_static")
        return y

    def forward_host(self, x):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty((x.shape[0], self.n_out), np.float32)
        self.eng._ok(self.eng.lib.ne_exl3_linear_host(C.byref(self.c), x.ctypes.data, x.shape[0], y.ctypes.data),
                     "ne_exl3_linear_host")
        return y


class EpExchange:
    """This rank's NVLink peer-memory exchange context (ne_ep_*): create, export the 64-byte IPC handle, connect with the
    handles of all ranks (rank order). One context serves every layer of a model."""

    def __init__(self, eng, rank, world, rows_cap, hidden, top_k):
        self.eng, self.rank, self.world = eng, rank, world
        self.ptr = eng.lib.ne_ep_create(rank, world, rows_cap, hidden, top_k)
        if not self.ptr:
            raise EngineError(eng.last_error())

    def handle(self):
        buf = C.create_string_buffer(64)
        self.eng._ok(self.eng.lib.ne_ep_handle(self.ptr, buf), "ne_ep_handle")
        return buf.raw

    def connect(self, handles):
        assert len(handles) == self.world and all(len(h) == 64 for h in handles)
        self.eng._ok(self.eng.lib.ne_ep_connect(self.ptr, C.create_string_buffer(b"".join(handles), 64 * self.world)), "ne_ep_connect")

    def free(self, barrier=None):
        """close the peers' mappings, let `barrier` (a callable, e.g. lambda: dist.barrier(group)) make sure every rank has
        done so, then free this rank's buffer: a buffer must not be freed while a peer still maps it"""
        if self.ptr:
            self.eng.lib.ne_ep_disconnect(self.ptr)
            if barrier is not None:
                barrier()
            self.eng.lib.ne_ep_free(self.ptr)
            self.ptr = None


def linear_multi(eng, linears, x, outs):
    """outs[i] = x @ W_i for up to 4 Exl3Linear objects that share the input width, in one launch chain
    (ne_exl3_linear_multi); x and outs are float32 device tensors the caller owns"""
    n = len(linears)
    ws = (Exl3WeightC * n)(*[l.c for l in linears])
    ys = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
    eng._ok(eng.lib.ne_exl3_linear_multi(ws, n, _dev(x), x.shape[0], ys, _stream()), "ne_exl3_linear_multi")
    return outs


class MoeBlock:
    """One MoE block on the device from a packgen-style tensor dict (or any mapping name -> (dtype, array)).
    expert slice [first, first + count) selects what this rank holds (expert parallel)."""

    def __init__(self, eng, tensors, layer=0, top_k=10, max_rows=16, expert_first=0, expert_count=None, device="cuda"):
        self.eng = eng
        pre = f"language_model.model.layers.{layer}.mlp."
        def g(n):
            a = tensors[pre + n][1]
            return a if hasattr(a, "data_ptr") else np.asarray(a)

        router = g("gate.weight")
        E, H = router.shape
        count = E if expert_count is None else expert_count
        # stacks that already hold only the local experts are taken whole
        sl = slice(None) if g("switch_mlp.gate_proj.trellis").shape[0] == count else slice(expert_first, expert_first + count)
        self.keep = []

        def dev(a):
            t = to_device_u16(a, device)
            self.keep.append(t)
            return t.data_ptr()

        d = MoeDescC()
        tr = g("switch_mlp.gate_proj.trellis")
        d.hidden, d.inter, d.experts, d.top_k = H, tr.shape[2] * 16, E, top_k
        d.k_expert = tr.shape[3] // 16
        d.expert_first, d.expert_count = expert_first, count
        d.router = dev(router)
        for name, fld in (("gate", "gate"), ("up", "up"), ("down", "down")):
            st = Exl3StackC(dev(g(f"switch_mlp.{name}_proj.trellis")[sl]), dev(g(f"switch_mlp.{name}_proj.suh")[sl]),
                            dev(g(f"switch_mlp.{name}_proj.svh")[sl]))
            setattr(d, fld, st)
        if pre + "shared_expert.gate_proj.trellis" in tensors:
            d.shared_gate_w = dev(g("shared_expert_gate.weight"))
            for name, fld in (("gate", "sh_gate"), ("up", "sh_up"), ("down", "sh_down")):
                t = g(f"shared_expert.{name}_proj.trellis")
                w = Exl3WeightC(dev(t), dev(g(f"shared_expert.{name}_proj.suh")), dev(g(f"shared_expert.{name}_proj.svh")),
                                t.shape[0] * 16, t.shape[1] * 16, t.shape[2] // 16)
                setattr(d, fld, w)
            d.k_shared = d.sh_gate.K
        self.desc, self.H, self.I, self.E, self.k, self.max_rows = d, H, d.inter, E, top_k, max_rows
        self.ptr = eng.lib.ne_moe_create(C.byref(d), max_rows)
        if not self.ptr:
            raise EngineError(f"ne_moe_create: {eng.last_error()}")

    def forward(self, x, out=None):
        torch = _torch()
        rows = x.shape[0]
        y = torch.empty((rows, self.H), dtype=torch.float32, device=x.device) if out is None else out
        self.eng._ok(self.eng.lib.ne_moe_forward(self.ptr, _dev(x), rows, _dev(y), _stream()), "ne_moe_forward")
        return y

    def forward_host(self, x, out=None):
        """x: numpy or pinned torch CPU float32 [rows, H]; returns numpy (or fills `out`)"""
        xp = x.data_ptr() if hasattr(x, "data_ptr") else np.ascontiguousarray(x, np.float32).ctypes.data
        rows = x.shape[0]
        y = np.empty((rows, self.H), np.float32) if out is None else out
        yp = y.data_ptr() if hasattr(y, "data_ptr") else y.ctypes.data
        self.eng._ok(self.eng.lib.ne_moe_forward_host(self.ptr, C.c_void_p(xp), rows, C.c_void_p(yp)), "ne_moe_forward_host")
        return y

    def stage(self, stage, x, y):
        self.eng._ok(self.eng.lib.ne_moe_stage(self.ptr, stage, _dev(x), x.shape[0], _dev(y), _stream()), f"ne_moe_stage({stage})")

    def forward_routed(self, x, route, out=None):
        torch = _torch()
        rows = x.shape[0]
        y = torch.empty((rows, self.H), dtype=torch.float32, device=x.device) if out is None else out
        self.eng._ok(self.eng.lib.ne_moe_forward_routed(self.ptr, _dev(x), _dev(route), rows, _dev(y), _stream()),
                     "ne_moe_forward_routed")
        return y

    def prefill(self, x, out=None):
        """n tokens at once through the sorted / grouped tcgen05 path (ne_moe_prefill); x [n, H] float32 on the device"""
        torch = _torch()
        n = x.shape[0]
        y = torch.empty((n, self.H), dtype=torch.float32, device=x.device) if out is None else out
        self.eng._ok(self.eng.lib.ne_moe_prefill(self.ptr, _dev(x), n, _dev(y), _stream()), "ne_moe_prefill")
        return y

    def route_rows(self, x, route_out):
        """the router alone on x; routes (ids, then float weights, as 32-bit words [rows, 2 top_k]) into the device tensor
        route_out, which may be a column slice of a wider row-major tensor (its row stride is passed on)"""
        ld = route_out.stride(0) if route_out.dim() == 2 else 0
        self.eng._ok(self.eng.lib.ne_moe_route(self.ptr, _dev(x), x.shape[0], C.c_void_p(route_out.data_ptr()), ld, _stream()), "ne_moe_route")
        return route_out

    def forward_ep_routed(self, x_all, route_all, own_row0, own_rows, out=None):
        """this rank's summand from the gathered rows and routes (ne_moe_forward_ep_routed); route_rows must have run on the
        own rows. x_all / route_all may be column slices of one packed row-major float32 / int32 tensor."""
        torch = _torch()
        rows = x_all.shape[0]
        y = torch.empty((rows, self.H), dtype=torch.float32, device=x_all.device) if out is None else out
        self.eng._ok(self.eng.lib.ne_moe_forward_ep_routed(self.ptr, C.c_void_p(x_all.data_ptr()), x_all.stride(0),
                                                           C.c_void_p(route_all.data_ptr()), route_all.stride(0), rows, own_row0, own_rows,
                                                           _dev(y), _stream()), "ne_moe_forward_ep_routed")
        return y

    def forward_ep_fused(self, xchg, x, out=None):
        """the whole expert-parallel block for this rank's rows x with both exchange steps over NVLink peer memory
        (ne_moe_forward_ep_fused); every rank calls with the same row count, in the same order"""
        torch = _torch()
        y = torch.empty_like(x) if out is None else out
        self.eng._ok(self.eng.lib.ne_moe_forward_ep_fused(self.ptr, xchg.ptr, _dev(x), x.shape[0], _dev(y), _stream()), "ne_moe_forward_ep_fused")
        return y

    def prefill_ep(self, x_all, own_row0, own_rows, out=None):
        """this rank's summand of the prefill output for the tokens of all ranks (ne_moe_prefill_ep)"""
        torch = _torch()
        n = x_all.shape[0]
        y = torch.empty((n, self.H), dtype=torch.float32, device=x_all.device) if out is None else out
        self.eng._ok(self.eng.lib.ne_moe_prefill_ep(self.ptr, _dev(x_all), n, own_row0, own_rows, _dev(y), _stream()),
                     "ne_moe_prefill_ep")
        return y

    # ---- the pieces of the all-to-all expert-parallel prefill (ijah_b200/ep.py puts the two exchanges between them)
    def prefill_home(self, x):
        """(y_shared [n, H], route int32 [n, 2k] = ids then f32 weight bits) of the rank's own tokens: routing and the
        shared expert, no routed expert (ne_moe_prefill_home)"""
        torch = _torch()
        n = x.shape[0]
        y = torch.empty((n, self.H), dtype=torch.float32, device=x.device)
        route = torch.empty((n, 2 * self.k), dtype=torch.int32, device=x.device)
        self.eng._ok(self.eng.lib.ne_moe_prefill_home(self.ptr, _dev(x), n, _dev(y), _dev(route), _stream()), "ne_moe_prefill_home")
        return y, route

    def prefill_routed(self, x_pairs, route_pairs):
        """weight * expert(x) for (token, slot) pairs routed elsewhere; route_pairs int32 [n, 2] = (expert id, f32 weight
        bits), every id one of this block's experts (ne_moe_prefill_routed)"""
        torch = _torch()
        n = x_pairs.shape[0]
        y = torch.empty((n, self.H), dtype=torch.float32, device=x_pairs.device)
        for i in range(0, n, 65535):  # one call takes at most 65535 rows
            m = min(65535, n - i)
            self.eng._ok(self.eng.lib.ne_moe_prefill_routed(self.ptr, _dev(x_pairs[i:i + m]), _dev(route_pairs[i:i + m]), m, _dev(y[i:i + m]),
                                                            _stream()), "ne_moe_prefill_routed")
        return y

    def pairs_by_owner(self, route, world):
        """(send_token int32 [n k], send_route int32 [n k, 2], pos int32 [n, k], counts int64 [world]) of a route array:
        its pairs in owner-rank order (ne_ep_pairs_by_owner)"""
        torch = _torch()
        if self.E % world:
            raise EngineError(f"pairs_by_owner: {self.E} experts do not split evenly over {world} ranks")
        n, k, dev = route.shape[0], self.k, route.device
        tok = torch.empty(n * k, dtype=torch.int32, device=dev)
        sr = torch.empty((n * k, 2), dtype=torch.int32, device=dev)
        pos = torch.empty((n, k), dtype=torch.int32, device=dev)
        counts = torch.empty(world, dtype=torch.int64, device=dev)
        self.eng._ok(self.eng.lib.ne_ep_pairs_by_owner(_dev(route), n, k, self.E // world, world, _dev(tok), _dev(sr), _dev(pos), _dev(counts),
                                                       _stream()), "ne_ep_pairs_by_owner")
        return tok, sr, pos, counts

    def gather_rows(self, src, index):
        """src[index] for rows of float32 (ne_rows_gather); index int32 on the device"""
        torch = _torch()
        out = torch.empty((index.shape[0], src.shape[1]), dtype=torch.float32, device=src.device)
        if index.shape[0]:
            self.eng._ok(self.eng.lib.ne_rows_gather(_dev(src), _dev(index), index.shape[0], src.shape[1], _dev(out), _stream()), "ne_rows_gather")
        return out

    def combine_slots(self, slots, pos, base, out=None):
        """y[t] = slots[pos[t, 0]] + .. + slots[pos[t, k-1]] + base[t], in that order (ne_slots_combine); pos int32 [n, k]"""
        torch = _torch()
        n, k = pos.shape
        y = torch.empty((n, slots.shape[1]), dtype=torch.float32, device=slots.device) if out is None else out
        self.eng._ok(self.eng.lib.ne_slots_combine(_dev(slots), _dev(pos), _dev(base), _dev(y), n, k, slots.shape[1], _stream()), "ne_slots_combine")
        return y

    def forward_ep(self, x_all, own_row0, own_rows, out=None):
        """this rank's summand of the block output for the rows of all ranks (ne_moe_forward_ep)"""
        torch = _torch()
        rows = x_all.shape[0]
        y = torch.empty((rows, self.H), dtype=torch.float32, device=x_all.device) if out is None else out
        self.eng._ok(self.eng.lib.ne_moe_forward_ep(self.ptr, _dev(x_all), rows, own_row0, own_rows, _dev(y), _stream()),
                     "ne_moe_forward_ep")
        return y

    def buffer(self, name, dtype=np.float32):
        """host copy of a named intermediate of the last run"""
        p, n = C.c_void_p(), C.c_uint64()
        self.eng._ok(self.eng.lib.ne_moe_buffer(self.ptr, name.encode(), C.byref(p), C.byref(n)), f"ne_moe_buffer({name})")
        out = np.empty(n.value // np.dtype(dtype).itemsize, dtype)
        self.eng._ok(self.eng.lib.ne_copy_to_host(out.ctypes.data, p, n.value), "ne_copy_to_host")
        return out

    def route(self, rows):
        r = self.buffer("route", np.uint32).reshape(rows, 2 * self.k)
        return r[:, :self.k].astype(np.int64), r[:, self.k:].copy().view(np.float32)

    def experts_gu(self, rows):
        out = np.empty((rows, self.k, 2, self.I), np.float32)
        self.eng._ok(self.eng.lib.ne_moe_experts_gu(self.ptr, rows, out.ctypes.data), "ne_moe_experts_gu")
        return out

    def last_bytes(self, rows):
        t, g, d, n = C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_int()
        self.eng._ok(self.eng.lib.ne_moe_last_bytes(self.ptr, rows, C.byref(t), C.byref(g), C.byref(d), C.byref(n)), "ne_moe_last_bytes")
        return dict(total=t.value, gateup=g.value, down=d.value, distinct_experts=n.value)

    def free(self):
        if self.ptr:
            self.eng.lib.ne_moe_free(self.ptr)
        self.ptr = None
