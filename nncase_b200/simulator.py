"""`Simulator`: runs a kmodel that carries a `cuda` module, with the surface of the reference's Python
interpreter binding (python/nncaseruntime/native/ffi.cpp:81-112: load_model, inputs_size, outputs_size,
get_input_desc, get_output_desc, set_input_tensor, get_input_tensor, get_output_tensor, set_profiling, run)
so that a test harness written for `nncase.Simulator` (tests/inference.py:68-86 of the reference) drives it
unchanged. Tensors are numpy arrays where the reference has RuntimeTensor (its `from_numpy` / `to_numpy` are
the identity here).

The kmodel's cuda function is executed by the library's native runtime function (nncb_program_* of the C
ABI: weights uploaded and every buffer planned at load_model, nothing allocated per run). With profiling on,
run() prints the per-operator table in the form of the reference's op_profile
(src/Native/src/runtime/stackvm/op_profile.cpp:25-111), timed with CUDA events.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import kmodel as K
from . import lib as L
from .kernels import Context, NncbError


@dataclass(frozen=True)
class TensorDesc:
    """tensor_desc of the reference: element type and shape (plus the quant param of u8 tensors)."""
    dtype: np.dtype
    shape: tuple
    scale: float = 1.0
    zero_point: int = 0


class Simulator:
    def __init__(self, device=0, ctx=None):
        self._ctx = ctx or Context(device)
        self._lib = self._ctx._lib
        self._prog = None
        self._inputs, self._outputs = [None], []
        self._profiling = False
        self.last_profile = None

    # ---- model -------------------------------------------------------------------------------------
    def load_model(self, data):
        model = K.read_kmodel(data)
        m, f = K.resolve_cuda_entry(model)
        mod = model["modules"][m]
        if mod["version"] != K.CUDA_MODULE_VERSION:
            raise NncbError(-38, f"cuda module version {mod['version']} is not supported")
        desc, rdata = mod["functions"][f]["sections"][".desc"], mod["sections"][".rdata"]
        self.close()
        h = C.c_void_p()
        L.check(self._lib.nncb_program_create(self._ctx._h, desc, len(desc), rdata, len(rdata), C.byref(h)))
        self._prog = h
        batch, nhwc, n_out = L._I32(), L._I32(), L._I32()
        chw = (L._I32 * 3)()
        L.check(self._lib.nncb_program_info(h, C.byref(batch), C.byref(nhwc), C.byref(chw), C.byref(n_out), None, None))
        c, hh, ww = chw[0], chw[1], chw[2]
        self._in_desc = TensorDesc(np.dtype(np.float32), (batch.value, hh, ww, c) if nhwc.value else (batch.value, c, hh, ww))
        self._out_desc = []
        for i in range(n_out.value):
            t, dt, sc, zp = L._I32(), L._I32(), L._F(), L._I32()
            hwc = (L._I32 * 3)()
            L.check(self._lib.nncb_program_output(h, i, C.byref(t)))
            L.check(self._lib.nncb_program_tensor(h, t.value, None, C.byref(hwc), C.byref(dt), C.byref(sc), C.byref(zp), None))
            self._out_desc.append(TensorDesc(np.dtype(np.float32 if dt.value == L.F32 else np.uint8),
                                             (batch.value, hwc[0], hwc[1], hwc[2]), sc.value, zp.value))
        self._inputs = [None]
        self._outputs = [None] * n_out.value

    @property
    def inputs_size(self):
        return 1

    @property
    def outputs_size(self):
        return len(self._out_desc)

    def get_input_desc(self, index):
        self._need_model()
        if index != 0:
            raise IndexError(index)
        return self._in_desc

    def get_output_desc(self, index):
        self._need_model()
        return self._out_desc[index]

    # ---- tensors ------------------------------------------------------------------------------------
    def set_input_tensor(self, index, tensor):
        d = self.get_input_desc(index)
        a = np.ascontiguousarray(tensor)
        if a.dtype != d.dtype or tuple(a.shape) != tuple(d.shape):
            raise NncbError(-22, f"input {index}: expected {d.dtype} {d.shape}, got {a.dtype} {tuple(a.shape)}")
        self._inputs[index] = a

    def get_input_tensor(self, index):
        return self._inputs[index]

    def get_output_tensor(self, index):
        if self._outputs[index] is None:
            raise NncbError(-61, "no output yet: call run() first")
        return self._outputs[index]

    def set_profiling(self, enabled):
        self._profiling = bool(enabled)

    # ---- execution ----------------------------------------------------------------------------------
    def run(self):
        self._need_model()
        if self._inputs[0] is None:
            raise NncbError(-22, "input 0 has not been set")
        outs = [np.empty(d.shape, d.dtype) for d in self._out_desc]
        ptrs = (C.c_void_p * len(outs))(*[o.ctypes.data for o in outs])
        L.check(self._lib.nncb_program_set_profiling(self._prog, int(self._profiling)))
        L.check(self._lib.nncb_program_run_host(self._ctx._h, self._prog, self._inputs[0].ctypes.data, ptrs, len(outs)))
        self._ctx.check_status()
        self._outputs = outs
        if self._profiling:
            need = L.check(self._lib.nncb_program_profile_text(self._prog, None, 0))
            buf = C.create_string_buffer(need + 1)
            L.check(self._lib.nncb_program_profile_text(self._prog, buf, need + 1))
            self.last_profile = buf.value.decode()
            print(self.last_profile)

    def launches_per_run(self):
        return int(self._lib.nncb_program_launches_per_call(self._prog))

    def close(self):
        if self._prog:
            self._lib.nncb_program_destroy(self._prog)
            self._prog = None

    def _need_model(self):
        if not self._prog:
            raise NncbError(-22, "no model loaded")

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
