"""ctypes driver of the REFERENCE's own C API (the `nncase_*` functions of src/Native/src/api.cpp, compiled into
oracle/_ref/libnncase_ref.so), bound the way its C# layer binds them
(src/Nncase.Simulator/Runtime/Interop/Native.cs:13-88). Test infrastructure: it lets the tests go
nncase_interp_load_model -> nncase_interp_get_entry_func -> nncase_func_invoke exactly as RTInterpreter does,
with the `cuda` plugin found by the reference's own loader."""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libnncase_ref.so")
PLUGIN = os.path.join(ROOT, "tests", "plugin_harness", "libnncase.simulator.cuda.so")
TYPECODE = {np.dtype(np.uint8): 0x06, np.dtype(np.float32): 0x0B, np.dtype(np.int8): 0x02, np.dtype(np.int32): 0x04}
NP_OF = {v: k for k, v in TYPECODE.items()}
MAP_READ, MAP_WRITE = 1, 2


class BufferSlice(C.Structure):
    _fields_ = [("buffer", C.c_void_p), ("start", C.c_uint32), ("size_bytes", C.c_uint32)]


class ReferenceError_(RuntimeError):
    def __init__(self, what, code):
        super().__init__(f"{what} failed with {code}")
        self.code = code


def available():
    return os.path.exists(REF) and os.path.exists(PLUGIN)


_lib = None


def lib():
    """The reference runtime. The plugin (linked against this very library, as a maintainer links it against
    Nncase.Runtime.Native) is loaded by path first so that the reference's loader finds it by soname."""
    global _lib
    if _lib is None:
        C.CDLL(PLUGIN)
        _lib = C.CDLL(REF)
    return _lib


def _chk(rc, what):
    if rc < 0:
        raise ReferenceError_(what, rc)
    return rc


def _make_tensor(arr):
    L = lib()
    arr = np.ascontiguousarray(arr)
    alloc, buf, hbuf = C.c_void_p(), C.c_void_p(), C.c_void_p()
    _chk(L.nncase_buffer_allocator_get_host(C.byref(alloc)), "get_host")
    _chk(L.nncase_buffer_allocator_alloc(alloc, C.c_uint32(arr.nbytes), None, C.byref(buf)), "alloc")
    _chk(L.nncase_buffer_as_host(buf, C.byref(hbuf)), "as_host")
    data, nbytes = C.c_void_p(), C.c_uint32()
    _chk(L.nncase_host_buffer_map(hbuf, MAP_WRITE, C.byref(data), C.byref(nbytes)), "map")
    C.memmove(data, arr.ctypes.data, arr.nbytes)
    _chk(L.nncase_host_buffer_unmap(hbuf), "unmap")
    dtype = C.c_void_p()
    _chk(L.nncase_dtype_create_prime(C.c_uint8(TYPECODE[arr.dtype]), C.byref(dtype)), "dtype")
    dims = (C.c_uint32 * arr.ndim)(*arr.shape)
    strides = (C.c_uint32 * arr.ndim)(*[s // arr.itemsize for s in arr.strides])
    sl = BufferSlice(buf.value, 0, arr.nbytes)
    t = C.c_void_p()
    _chk(L.nncase_tensor_create(dtype, dims, arr.ndim, strides, arr.ndim, C.byref(sl), C.byref(t)), "tensor_create")
    return t


def _read_tensor(t):
    L = lib()
    n = C.c_uint32(8)
    dims = (C.c_uint32 * 8)()
    _chk(L.nncase_tensor_get_dims(t, dims, C.byref(n)), "get_dims")
    shape = tuple(dims[i] for i in range(n.value))
    dt = C.c_void_p()
    _chk(L.nncase_tensor_get_dtype(t, C.byref(dt)), "get_dtype")
    code = L.nncase_dtype_get_typecode(dt)
    sl = BufferSlice()
    _chk(L.nncase_tensor_get_buffer(t, C.byref(sl)), "get_buffer")
    hbuf = C.c_void_p()
    _chk(L.nncase_buffer_as_host(C.c_void_p(sl.buffer), C.byref(hbuf)), "as_host")
    data, nbytes = C.c_void_p(), C.c_uint32()
    _chk(L.nncase_host_buffer_map(hbuf, MAP_READ, C.byref(data), C.byref(nbytes)), "map")
    out = np.empty(shape, NP_OF[code])
    C.memmove(out.ctypes.data, data.value + sl.start, out.nbytes)
    _chk(L.nncase_host_buffer_unmap(hbuf), "unmap")
    return out


class Interpreter:
    """RTInterpreter.Create / LoadModel / Entry.Invoke (src/Nncase.Simulator/Runtime/Interop/RTInterpreter.cs:58-87)."""

    def __init__(self):
        self._h = C.c_void_p()
        _chk(lib().nncase_interp_create(C.byref(self._h)), "nncase_interp_create")
        self._model = None

    def load_model(self, data, copy=True):
        self._model = C.create_string_buffer(bytes(data), len(data))  # must outlive the interpreter when not copied
        _chk(lib().nncase_interp_load_model(self._h, self._model, C.c_uint32(len(data)), C.c_bool(copy)),
             "nncase_interp_load_model")

    def invoke(self, *inputs):
        L = lib()
        fn = C.c_void_p()
        _chk(L.nncase_interp_get_entry_func(self._h, C.byref(fn)), "nncase_interp_get_entry_func")
        n = C.c_uint32()
        _chk(L.nncase_func_get_params_size(fn, C.byref(n)), "nncase_func_get_params_size")
        assert n.value == len(inputs)
        params = (C.c_void_p * len(inputs))(*[_make_tensor(x) for x in inputs])
        res = C.c_void_p()
        _chk(L.nncase_func_invoke(fn, params, C.c_uint32(len(inputs)), C.byref(res)), "nncase_func_invoke")
        is_t = C.c_bool()
        _chk(L.nncase_value_is_tensor(res, C.byref(is_t)), "value_is_tensor")
        if is_t.value:
            return _read_tensor(res)
        cnt = C.c_uint32(64)
        fields = (C.c_void_p * 64)()
        _chk(L.nncase_tuple_get_fields(res, fields, C.byref(cnt)), "tuple_get_fields")
        return [_read_tensor(C.c_void_p(fields[i])) for i in range(cnt.value)]

    def close(self):
        if self._h:
            lib().nncase_interp_free(self._h)
            self._h = None
