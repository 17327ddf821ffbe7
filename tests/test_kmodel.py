"""kmodels with a `cuda` module: the writer against the REFERENCE's own loader and interpreter, and the
library's Simulator.

The reference runtime (oracle/_ref/libnncase_ref.so = its native sources compiled in simulator mode) parses
the bytes nncase_b200.kmodel writes, activates the plugin for module kind "cuda" through its own loader and
runs the entry function through nncase_func_invoke -- directly, or through a StackVM `main` that EXTCALLs the
cuda function (src/Native/src/runtime/stackvm/ops/control.cpp:25-78). Results: bit-exact against the oracle.
"""
import struct

import numpy as np
import pytest

from nncase_b200 import builder, kmodel, networks
from oracle import program as oprog

import ref_runtime as RR


def _config1(hw=28):
    g = networks.single_conv(seed=1001, c=64, oc=64, hw=hw)
    cal = [np.random.default_rng(3001 + i).uniform(-1, 1, (1, 64, hw, hw)).astype(np.float32) for i in range(8)]
    return builder.build_program(g, cal)


# ---- CPU: format ------------------------------------------------------------------------------------------
def test_writer_reader_round_trip():
    prog = _config1()
    for via in (False, True):
        data = kmodel.write_kmodel(prog, 2, via_stackvm=via)
        ident, version, _, _, n_mod, e_mod, e_fn, _ = struct.unpack_from("<8I", data, 0)
        assert ident == int.from_bytes(b"LDMK", "little") and version == 7 and (e_mod, e_fn) == (0, 0)
        m = kmodel.read_kmodel(data)
        assert [x["kind"] for x in m["modules"]] == (["stackvm", "cuda"] if via else ["cuda"])
        mi, fi = kmodel.resolve_cuda_entry(m)
        cuda = m["modules"][mi]
        desc = cuda["functions"][fi]["sections"][".desc"]
        magic, ver, batch, n_t, n_ops = struct.unpack_from("<5I", desc, 0)
        assert (magic, ver, batch) == (kmodel.DESC_MAGIC, 1, 2)
        assert n_t == len(prog["tensors"]) and n_ops == len(prog["ops"])
        # the weights are in .rdata byte for byte, 16-byte aligned in the file
        w = [o for o in prog["ops"] if o["op"] == "conv"][0]["w"].tobytes()
        assert w in cuda["sections"][".rdata"]
        assert data.index(w) % 16 == 0
        if via:
            vm = m["modules"][0]
            assert set(vm["sections"]) == {".text", ".rdata", ".custom_calls"}
            assert vm["sections"][".text"] == bytes([40, 2, 0, 0, 0, 0, 2, 1, 0, 0, 0, 96, 1, 0, 0, 93])


def test_reader_rejects_foreign_bytes():
    good = kmodel.write_kmodel(_config1(), 1)
    with pytest.raises(ValueError):
        kmodel.read_kmodel(b"not a kmodel at all, but long enough to hold a header")
    v5 = bytearray(good)
    struct.pack_into("<I", v5, 4, 5)          # the version of the kmodels bundled with the reference's benchmark
    with pytest.raises(ValueError, match="version 5"):
        kmodel.read_kmodel(bytes(v5))


def test_reference_loader_parses_the_kmodel_and_reaches_the_plugin():
    """Without a GPU the load fails -- inside the plugin's module initialisation (no device, no fallback), which
    is reached only if the reference's loader accepted every header before it; wrong identifier and wrong
    version are refused by the reference itself with its own error codes."""
    import torch
    if not RR.available():
        pytest.skip("reference runtime / plugin not built")
    data = kmodel.write_kmodel(_config1(), 1)
    bad_id = bytearray(data)
    bad_id[0] ^= 0xFF
    it = RR.Interpreter()
    with pytest.raises(RR.ReferenceError_) as e:
        it.load_model(bytes(bad_id))
    assert e.value.code == -0x01      # nncase_errc::invalid_model_indentifier
    v5 = bytearray(data)
    struct.pack_into("<I", v5, 4, 5)
    with pytest.raises(RR.ReferenceError_) as e:
        it.load_model(bytes(v5))
    assert e.value.code == -0x03      # nncase_errc::invalid_model_version
    if torch.cuda.is_available():
        it.load_model(data)
    else:
        with pytest.raises(RR.ReferenceError_) as e:
            it.load_model(data)
        assert e.value.code == -5     # -EIO from nncb_context_create, carried through result<>
    it.close()


# ---- GPU: execution ---------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("via_stackvm", [False, True])
def test_config1_through_the_reference_interpreter(ctx, via_stackvm):
    if not RR.available():
        pytest.skip("reference runtime / plugin not built")
    prog = _config1(56)
    x = np.random.default_rng(2001).uniform(-1, 1, (1, 64, 56, 56)).astype(np.float32)
    want, _ = oprog.run_program(prog, x)
    it = RR.Interpreter()
    it.load_model(kmodel.write_kmodel(prog, 1, via_stackvm=via_stackvm), copy=not via_stackvm)
    got = it.invoke(x)
    assert got.dtype == np.uint8 and np.array_equal(got, want)
    assert np.array_equal(it.invoke(x), want)  # a second call on the planned buffers
    it.close()


@pytest.mark.gpu
def test_resnet50v2_through_the_reference_interpreter(ctx):
    if not RR.available():
        pytest.skip("reference runtime / plugin not built")
    graph = networks.resnet50v2(1003)
    cal = [np.random.default_rng(3003 + i).normal(0, 1, (1, 3, 224, 224)).astype(np.float32) for i in range(16)]
    prog = builder.build_program(graph, cal, device=ctx.device)
    x = np.random.default_rng(2003).normal(0, 1, (1, 3, 224, 224)).astype(np.float32)
    want, _ = oprog.run_program(prog, x)
    it = RR.Interpreter()
    it.load_model(kmodel.write_kmodel(prog, 1, via_stackvm=True))
    got = it.invoke(x)
    assert got.dtype == np.float32 and got.shape == (1, 1, 1, 1000) and np.array_equal(got, want)
    it.close()


@pytest.mark.gpu
def test_simulator_matches_the_oracle_and_prints_a_profile(ctx, capsys):
    from nncase_b200.simulator import Simulator
    graph = networks.mobilenetv2(1002)
    cal = [(np.random.default_rng(3002 + i).uniform(0, 1, (1, 224, 224, 3)).astype(np.float32) - 0.5) / 0.5
           for i in range(4)]
    prog = builder.build_program(graph, cal, device=ctx.device)
    x = (np.random.default_rng(2002).uniform(0, 1, (3, 224, 224, 3)).astype(np.float32) - 0.5) / 0.5
    want, _ = oprog.run_program(prog, x)
    sim = Simulator(ctx=ctx)
    sim.load_model(kmodel.write_kmodel(prog, 3))
    assert sim.inputs_size == 1 and sim.outputs_size == 1
    assert sim.get_input_desc(0).shape == (3, 224, 224, 3) and sim.get_output_desc(0).dtype == np.float32
    sim.set_input_tensor(0, x)
    sim.run()
    assert np.array_equal(sim.get_output_tensor(0), want)
    sim.set_profiling(True)
    sim.run()
    assert np.array_equal(sim.get_output_tensor(0), want)
    text = sim.last_profile
    assert "stack OPs timeline" in text and "cuda OPs profile" in text and "|conv2d" in text and "|total" in text
    assert text in capsys.readouterr().out
    n_ops = len(prog["ops"])
    assert sum(1 for line in text.split("cuda OPs profile")[0].splitlines() if line.startswith("|") and "---" not in line) == n_ops + 1
    assert sim.launches_per_run() >= n_ops
    with pytest.raises(Exception):
        sim.set_input_tensor(0, x[:1])
    sim.close()


@pytest.mark.gpu
def test_simulator_several_outputs_and_stackvm_entry(ctx):
    """YOLOv8s: Slice / Concat / Upsample records, SiLU tables from .rdata, six u8 outputs."""
    from nncase_b200.simulator import Simulator
    graph = networks.yolov8s(1004, image=320)
    cal = [np.random.default_rng(3004 + i).uniform(0, 1, (1, 3, 320, 320)).astype(np.float32) for i in range(2)]
    prog = builder.build_program(graph, cal, device=ctx.device)
    x = np.random.default_rng(2004).uniform(0, 1, (2, 3, 320, 320)).astype(np.float32)
    _, tens = oprog.run_program(prog, x)
    sim = Simulator(ctx=ctx)
    sim.load_model(kmodel.write_kmodel(prog, 2, via_stackvm=True))
    assert sim.outputs_size == 6
    sim.set_input_tensor(0, x)
    sim.run()
    for i, name in enumerate(prog["outputs"]):
        assert np.array_equal(sim.get_output_tensor(i), tens[name]), name
    if RR.available():
        it = RR.Interpreter()
        it.load_model(kmodel.write_kmodel(prog, 2, via_stackvm=True))
        outs = it.invoke(x)
        assert len(outs) == 6
        for got, name in zip(outs, prog["outputs"]):
            assert np.array_equal(got, tens[name]), name
        it.close()
    sim.close()


@pytest.mark.gpu
def test_malformed_descriptors_are_refused(ctx):
    """nncb_program_create on damaged sections: an error code, never a crash or an out-of-bounds read."""
    import ctypes as C

    from nncase_b200 import lib as L
    desc, rdata, _ = kmodel.serialize_program(_config1(), 1)

    def create(d, r):
        h = C.c_void_p()
        rc = ctx._lib.nncb_program_create(ctx._h, d, len(d), r, len(r), C.byref(h))
        if rc == 0:
            ctx._lib.nncb_program_destroy(h)
        return rc

    assert create(desc, rdata) == 0
    assert create(desc[:40], rdata) == -22                        # truncated header
    assert create(b"XXXX" + desc[4:], rdata) == -22               # wrong magic
    assert create(desc[:4] + struct.pack("<I", 9) + desc[8:], rdata) == -38   # unknown version
    assert create(desc[:-8], rdata) == -22                        # operator table cut short
    assert create(desc, rdata[:100]) == -22                       # weights outside .rdata
    bad_idx = bytearray(desc)
    n_t = struct.unpack_from("<I", desc, 12)[0]
    op0 = 48 + 4 + n_t * 24                                       # header, one output index, tensor table
    struct.pack_into("<i", bad_idx, op0 + 160 + 32, 1000)         # second op (the convolution): input tensor index
    assert create(bytes(bad_idx), rdata) == -22
