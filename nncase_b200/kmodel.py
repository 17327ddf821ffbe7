"""kmodel (KMDL version 7) writer and reader for models that carry a `cuda` module.

The reference's compiler writes kmodels from C# (src/Nncase.CodeGen/CodeGen/LinkedModel.cs:27-170,
structs in KModelTypes.cs:17-65) and its native runtime reads them
(src/Native/include/nncase/runtime/model.h:38-99, src/Native/src/runtime/interpreter.cpp:33-65,
runtime_module.cpp:124-152, runtime_function.cpp:126-150, section.cpp:20-46). This module is the
module builder's serializer for the `cuda` module kind, in Python where the reference's is C#:

  model_header | module* ;  module = module_header | function* | section*
  function = function_header | parameter types | return type | section*
  section  = section_header | padding to the body's alignment | body | padding to 8

A model is written either with the cuda function as the entry point, or -- the way the reference's
compiler links a callee of another module kind -- behind a StackVM `main` whose bytecode is
LDARG_0, LDC_I4 function id, LDC_I4 module id, EXTCALL 1 (not a prim function), RET
(opcodes: src/Native/include/nncase/runtime/stackvm/opcode.h:26-127; the call:
src/Native/src/runtime/stackvm/ops/control.cpp:25-78; how the C# code generator emits it:
modules/Nncase.Modules.StackVM/CodeGen/StackVM/CodegenVisitor.cs:311-315,470-476).

The `cuda` module (kind "cuda", version 1):
  module section ".rdata"   weights (u8|i8 OHWI), weight zero points (i32), multipliers (f32), bias (f32),
                            activation tables (256 x u8); every blob 16-byte aligned
  function section ".desc"  the launch list: header, output tensor indices, tensor table, operator records
                            (struct layouts below = DescHeader / DescTensor / DescOp of csrc/program.cu)
"""
import struct

import numpy as np

MODEL_IDENTIFIER = int.from_bytes(b"LDMK", "little")  # the multi-character constant 'KMDL'
MODEL_VERSION = 7
MODEL_HAS_NO_ENTRY = 0xFFFFFFFF
DESC_MAGIC, DESC_VERSION = 0x4455434E, 1
CUDA_MODULE_VERSION = 1
STACKVM_MODULE_VERSION = 1

# typecodes (src/Native/include/nncase/runtime/typecodes.def) and type signature tokens
# (src/Native/include/nncase/runtime/type_serializer.h:23-30)
DT_U8, DT_F32 = 0x06, 0x0B
SIG_TENSOR, SIG_TUPLE, SIG_END = 2, 3, 0xFF
# StackVM opcodes used by the trampoline
OP_LDC_I4, OP_LDARG_0, OP_RET, OP_EXTCALL = 2, 40, 93, 96

(K_QUANT_INPUT, K_CONV, K_MAXPOOL, K_REQUANT, K_ADD, K_SLICE, K_CONCAT_PART, K_UPSAMPLE, K_GAP) = range(9)
INF = float("inf")


class _Writer:
    """Sequential writer with the reference serializer's habits (LinkedModel.cs): headers are skipped and
    patched once the size is known, bodies are aligned on the absolute stream position, every function,
    section and module ends 8-aligned."""

    def __init__(self):
        self.buf = bytearray()

    def pos(self):
        return len(self.buf)

    def write(self, b):
        self.buf += b

    def align(self, n):
        pad = (-len(self.buf)) % n
        self.buf += b"\0" * pad
        return pad

    def patch(self, pos, b):
        self.buf[pos:pos + len(b)] = b


def _kind(name, width=16):
    b = name.encode()
    assert 0 < len(b) <= width
    return b + b"\0" * (width - len(b))


def _write_section(w, name, body, align=8):
    """section_header {char name[16]; u32 flags, reserved; u64 size, body_start, body_size, memory_size} | body;
    body_start is the padding between the end of the header and the body (section.cpp:20-46)."""
    start = w.pos()
    w.write(b"\0" * 56)
    pad = w.align(align)
    w.write(body)
    w.align(8)
    w.patch(start, _kind(name) + struct.pack("<IIQQQQ", 0, 0, w.pos() - start, pad, len(body), len(body)))


def _tensor_type(dtype_code, shape):
    out = struct.pack("<BBB", SIG_TENSOR, dtype_code, 1)
    for d in shape:
        out += struct.pack("<BI", 1, int(d))  # dim_fixed, value
    return out + struct.pack("<B", SIG_END)


def _tuple_type(types):
    return struct.pack("<B", SIG_TUPLE) + b"".join(types) + struct.pack("<B", SIG_END)


def _write_function(w, param_types, return_type, sections, entrypoint=0, text_size=0):
    """function_header {u32 parameters, sections; u64 entrypoint, text_size, size} | parameter types | return
    type | sections (no padding between the types and the first section header: runtime_function.cpp:126-150)."""
    start = w.pos()
    w.write(b"\0" * 32)
    for t in param_types:
        w.write(t)
    w.write(return_type)
    for name, body, align in sections:
        _write_section(w, name, body, align)
    w.align(8)
    w.patch(start, struct.pack("<IIQQQ", len(param_types), len(sections), entrypoint, text_size, w.pos() - start))


def _write_module(w, kind, version, functions, sections):
    """module_header {char kind[16]; u32 version, sections, functions, reserved; u64 size} | functions | sections."""
    start = w.pos()
    w.write(b"\0" * 40)
    for fn in functions:
        _write_function(w, *fn)
    for name, body, align in sections:
        _write_section(w, name, body, align)
    w.align(8)
    w.patch(start, _kind(kind) + struct.pack("<IIIIQ", version, len(sections), len(functions), 0, w.pos() - start))


# ---- the cuda function's descriptor ---------------------------------------------------------------
class _Rdata:
    def __init__(self):
        self.buf = bytearray()

    def add(self, arr):
        if arr is None:
            return -1
        self.buf += b"\0" * ((-len(self.buf)) % 16)
        off = len(self.buf)
        self.buf += np.ascontiguousarray(arr).tobytes()
        return off


def serialize_program(program, batch):
    """A quantized program (nncase_b200.builder.build_program) -> (desc bytes, rdata bytes, io) where io
    describes the function's parameter and results for the kmodel's type signatures."""
    T = program["tensors"]
    names = list(T)
    index = {n: i for i, n in enumerate(names)}
    rd = _Rdata()
    ops = []

    def rec(kind, name, ints=(), floats=()):
        ints, floats = list(ints), list(floats)
        assert len(ints) <= 24 and len(floats) <= 8
        ints += [0] * (24 - len(ints))
        floats += [0.0] * (8 - len(floats))
        nm = name.encode()[:27]
        ops.append(struct.pack("<I28s24i8f", kind, nm, *[int(v) for v in ints], *[float(v) for v in floats]))

    qin = None
    for op in program["ops"]:
        k = op["op"]
        if k == "quantize_input":
            qin = op
            pad = op.get("pad", (0, 0, 0, 0))
            rec(K_QUANT_INPUT, "input", [index[op["out"]], op["c"], op["c_pad"], int(bool(op.get("s2d"))), *pad])
        elif k == "conv":
            w = op["w"]
            oc, kh, kw, _ = w.shape
            f32 = bool(op.get("f32_out"))
            cq = op.get("conv_qp")
            ints = [index[op["in"]], index[op["out"]], index[op["res"]] if op.get("res") else -1,
                    index[op["y2"]] if op.get("y2") else -1, oc, kh, kw, *op["stride"], *op["pad"], *op["dil"],
                    op["groups"], int(w.dtype == np.int8), int(f32), rd.add(op.get("lut")), rd.add(w),
                    rd.add(None if op["w_zp"] is None else np.asarray(op["w_zp"], np.int32)),
                    rd.add(np.asarray(op["mult"], np.float32)), rd.add(np.asarray(op["bias"], np.float32)),
                    0 if f32 else cq.zero_point]
            rec(K_CONV, op["name"], ints, [op["clamp"][0], op["clamp"][1], 1.0 if f32 else cq.scale])
        elif k == "maxpool":
            rec(K_MAXPOOL, "maxpool", [index[op["in"]], index[op["out"]], *op["k"], *op["stride"], *op["pad"]])
        elif k == "requant":
            rec(K_REQUANT, "clamp", [index[op["in"]], index[op["out"]]], list(op["clamp"]))
        elif k == "add":
            rec(K_ADD, "add", [index[op["a"]], index[op["b"]], index[op["out"]]])
        elif k == "slice":
            rec(K_SLICE, "slice", [index[op["in"]], index[op["out"]], op["begin"], op["end"]])
        elif k == "concat":
            off = 0
            for name in op["ins"]:
                rec(K_CONCAT_PART, "concat", [index[name], index[op["out"]], off])
                off += T[name]["shape"][2]
        elif k == "upsample":
            rec(K_UPSAMPLE, "upsample", [index[op["in"]], index[op["out"]], op["factor"]])
        elif k == "gap":
            rec(K_GAP, "global_mean", [index[op["in"]], index[op["out"]]])
        else:
            raise ValueError(f"operator {k} has no record in the cuda descriptor")
    if qin is None:
        raise ValueError("a program starts with its input stage")
    # input geometry: the f32 tensor the caller passes
    tin = T[program["input"]]
    pad = qin.get("pad", (0, 0, 0, 0))
    h, w, _ = tin["shape"]
    if qin.get("s2d"):
        in_h, in_w = (h - pad[0] - pad[1]) * 2, (w - pad[2] - pad[3]) * 2
    else:
        in_h, in_w = h, w
    nhwc = int(bool(qin.get("nhwc")))
    outs = [index[n] for n in program.get("outputs", [program["output"]])]
    header = struct.pack("<12I", DESC_MAGIC, DESC_VERSION, batch, len(names), len(ops), index[program["input"]], nhwc,
                         qin["c"], in_h, in_w, len(outs), 0)
    tens = b""
    for n in names:
        t = T[n]
        hh, ww, cc = t["shape"]
        qp = t["qp"]
        tens += struct.pack("<4Iif", hh, ww, cc, 1 if t["dtype"] == "f32" else 0, qp.zero_point if qp else 0,
                            qp.scale if qp else 1.0)
    desc = header + struct.pack(f"<{len(outs)}I", *outs) + tens + b"".join(ops)
    in_shape = (batch, in_h, in_w, qin["c"]) if nhwc else (batch, qin["c"], in_h, in_w)
    out_types = []
    for n in program.get("outputs", [program["output"]]):
        hh, ww, cc = T[n]["shape"]
        out_types.append((DT_F32 if T[n]["dtype"] == "f32" else DT_U8, (batch, hh, ww, cc)))
    return desc, bytes(rd.buf), dict(in_shape=in_shape, out_types=out_types)


def write_kmodel(program, batch, via_stackvm=True):
    """Bytes of a kmodel whose entry runs `program` on the cuda module for `batch` images. With via_stackvm the
    entry is a StackVM `main` (module 0) that EXTCALLs function 0 of the cuda module (module 1)."""
    desc, rdata, io = serialize_program(program, batch)
    ptype = _tensor_type(DT_F32, io["in_shape"])
    rtypes = [_tensor_type(dt, shp) for dt, shp in io["out_types"]]
    rtype = rtypes[0] if len(rtypes) == 1 else _tuple_type(rtypes)
    cuda_fn = ([ptype], rtype, [(".desc", desc, 8)])
    cuda_mod = ("cuda", CUDA_MODULE_VERSION, [cuda_fn], [(".rdata", rdata, 16)])
    if not via_stackvm:
        modules = [cuda_mod]
    else:
        text = (struct.pack("<B", OP_LDARG_0) + struct.pack("<Bi", OP_LDC_I4, 0) + struct.pack("<Bi", OP_LDC_I4, 1) +
                struct.pack("<BHB", OP_EXTCALL, 1, 0) + struct.pack("<B", OP_RET))
        main = ([ptype], rtype, [], 0, len(text))
        # ".custom_calls": u32 count of module kinds whose custom calls the module uses (none here)
        vm_mod = ("stackvm", STACKVM_MODULE_VERSION, [main],
                  [(".text", text, 8), (".rdata", b"\0" * 8, 8), (".custom_calls", struct.pack("<I", 0), 8)])
        modules = [vm_mod, cuda_mod]
    w = _Writer()
    w.write(struct.pack("<8I", MODEL_IDENTIFIER, MODEL_VERSION, 0, 16, len(modules), 0, 0, 0))
    for m in modules:
        _write_module(w, *m)
    return bytes(w.buf)


# ---- reader -------------------------------------------------------------------------------------------
def _sections(buf, pos, count):
    out = {}
    for _ in range(count):
        name = bytes(buf[pos:pos + 16]).split(b"\0")[0].decode()
        flags, _r, size, start, bsize, _m = struct.unpack_from("<IIQQQQ", buf, pos + 16)
        body0 = pos + 56 + start
        out[name] = bytes(buf[body0:body0 + bsize])
        pos += size
    return out, pos


def _skip_type(buf, pos):
    tok = buf[pos]
    pos += 1
    if tok == SIG_TENSOR:
        pos += 1  # element typecode (primitive types only here)
        if buf[pos] == 0:
            return pos + 1
        pos += 1
        while buf[pos] != SIG_END:
            pos += 5 if buf[pos] == 1 else 1
        return pos + 1
    if tok == SIG_TUPLE:
        while buf[pos] != SIG_END:
            pos = _skip_type(buf, pos)
        return pos + 1
    return pos


def read_kmodel(data):
    """Parses a kmodel into {entry: (module, function), modules: [{kind, version, sections, functions:
    [{parameters, entrypoint, text_size, sections}]}]}; raises ValueError on anything that is not a
    version-7 kmodel."""
    buf = memoryview(bytes(data))
    if len(buf) < 32:
        raise ValueError("not a kmodel: shorter than its header")
    ident, version, _flags, _align, n_mod, e_mod, e_fn, _ = struct.unpack_from("<8I", buf, 0)
    if ident != MODEL_IDENTIFIER:
        raise ValueError("not a kmodel: bad identifier")
    if version != MODEL_VERSION:
        raise ValueError(f"kmodel version {version}; this reader (like the runtime) takes version {MODEL_VERSION}")
    pos, modules = 32, []
    for _ in range(n_mod):
        kind = bytes(buf[pos:pos + 16]).split(b"\0")[0].decode()
        mver, n_sec, n_fn, _r, msize = struct.unpack_from("<IIIIQ", buf, pos + 16)
        p, fns = pos + 40, []
        for _ in range(n_fn):
            n_par, f_sec, entry, tsize, fsize = struct.unpack_from("<IIQQQ", buf, p)
            q = p + 32
            for _ in range(n_par + 1):
                q = _skip_type(buf, q)
            secs, _ = _sections(buf, q, f_sec)
            fns.append(dict(parameters=n_par, entrypoint=entry, text_size=tsize, sections=secs))
            p += fsize
        secs, _ = _sections(buf, p, n_sec)
        modules.append(dict(kind=kind, version=mver, sections=secs, functions=fns))
        pos += msize
    entry = None if e_mod == MODEL_HAS_NO_ENTRY else (e_mod, e_fn)
    return dict(entry=entry, modules=modules)


def resolve_cuda_entry(model):
    """(module index, function index) of the cuda function the model's entry runs: the entry itself, or the
    callee of a StackVM trampoline (LDARG_0, LDC_I4 f, LDC_I4 m, EXTCALL, RET)."""
    if model["entry"] is None:
        raise ValueError("the kmodel has no entry function")
    m, f = model["entry"]
    mod = model["modules"][m]
    if mod["kind"] == "cuda":
        return m, f
    if mod["kind"] != "stackvm":
        raise ValueError(f"entry module of kind {mod['kind']!r} is not supported")
    fn = mod["functions"][f]
    text = mod["sections"][".text"][fn["entrypoint"]:fn["entrypoint"] + fn["text_size"]]
    want = struct.calcsize("<BBiBiBHBB")
    if len(text) != want:
        raise ValueError("the StackVM entry is not a call trampoline into the cuda module")
    o0, o1, fid, o2, mid, o3, args, prim, o4 = struct.unpack("<BBiBiBHBB", text)
    if (o0, o1, o2, o3, o4, args, prim) != (OP_LDARG_0, OP_LDC_I4, OP_LDC_I4, OP_EXTCALL, OP_RET, 1, 0):
        raise ValueError("the StackVM entry is not a call trampoline into the cuda module")
    if model["modules"][mid]["kind"] != "cuda":
        raise ValueError("the StackVM entry calls a module that is not of kind cuda")
    return mid, fid
