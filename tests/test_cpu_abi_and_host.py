"""CPU-side checks: the shared libraries load and export every symbol the headers declare,
descriptors are packed as the MLIR ABI says, argument validation rejects bad calls without
touching a GPU, the tile table answers, and batch sharding is consistent."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parents[1]


def declared_symbols(header: Path):
    text = header.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"HOM_EXPORT\s+[\w\s\*]+?\b(\w+)\s*\(", text)
    return sorted(set(names))


def test_runner_library_exports_every_declared_symbol(pkg, hom):
    names = declared_symbols(REPO / "include" / "hom_nvgpu_runner_utils.h")
    assert len(names) >= 45
    for n in names:
        assert hasattr(hom.lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(pkg.EXPORTED_SYMBOLS)
    # the C++ allocation hook that harnesses written for the reference use
    assert ctypes.c_void_p.in_dll(hom.lib, "nvgpuAllocer") is not None


def test_library_keeps_the_reference_file_name(pkg):
    assert pkg.RUNNER_LIB.name == "libhands_on_mlir_nvgpu_runner_utils.so"


def test_replay_library_exports_every_declared_symbol(pkg, hom):
    lib = ctypes.CDLL(str(pkg.REPLAY_LIB))
    for n in declared_symbols(REPO / "include" / "hom_bert_replay.h"):
        assert hasattr(lib, n), n


def test_memref_descriptor_layout(pkg):
    m = pkg.MemRef(0x1000, (2, 3, 8))
    words = list(m._words)
    assert words == [0x1000, 0x1000, 0, 2, 3, 8, 24, 8, 1]
    rank, ptr = m.args
    assert rank.value == 3 and ptr.value == ctypes.addressof(m._words)
    assert ctypes.sizeof(pkg.UnrankedMemRef) == 16


def test_memref_of_numpy_backed_tensor(pkg):
    import torch
    t = torch.zeros((4, 5, 6), dtype=torch.float16)[:, 1:3]
    m = pkg.MemRef.of(t)
    assert m.shape == [4, 2, 6] and m.strides == [30, 6, 1] and m.data_ptr == t.data_ptr()


def _host_memref(pkg, shape, itemsize=2):
    buf = np.zeros(int(np.prod(shape)) * itemsize + 16, dtype=np.uint8)
    addr = (buf.ctypes.data + 15) & ~15
    return pkg.MemRef(addr, shape, keepalive=buf)


def test_validation_rejects_without_launching(pkg, hom):
    """Malformed calls record an error and return; nothing is launched (no GPU needed)."""
    before = hom.launch_count()
    A, B, D = _host_memref(pkg, (1, 128, 64)), _host_memref(pkg, (1, 72, 64)), _host_memref(pkg, (1, 128, 64))
    with pytest.raises(pkg.HomError) as e:
        hom.cutlassGemmF16(A, B, D, D)
    assert e.value.code == 1 and "inner dimensions" in e.value.message
    with pytest.raises(pkg.HomError) as e:
        hom.cutlassGemmF16(A, _host_memref(pkg, (2, 64, 64)), D, D)
    assert e.value.code == 2
    with pytest.raises(pkg.HomError) as e:
        hom.cutlassGemmF16(A, _host_memref(pkg, (1, 64, 64)), D, D, activation=3)
    assert e.value.code == 2
    with pytest.raises(pkg.HomError):
        hom.cutlassGemmF16(None, B, D, D)
    with pytest.raises(pkg.HomError):
        hom.nvteGemmF16(A, B, D, D, alpha=2.0)
    with pytest.raises(pkg.HomError):
        hom.nvteLayernormF16(_host_memref(pkg, (8,)), 1e-5)
    with pytest.raises(pkg.HomError):
        hom.elementwise("Add", "F16", _host_memref(pkg, (2, 3)), _host_memref(pkg, (3, 3)),
                        _host_memref(pkg, (2, 3)))
    with pytest.raises(pkg.HomError):  # A may not broadcast
        hom.elementwise("Add", "F16", _host_memref(pkg, (1, 3)), _host_memref(pkg, (2, 3)),
                        _host_memref(pkg, (2, 3)))
    with pytest.raises(pkg.HomError):
        hom.gather("F16", _host_memref(pkg, (2, 3), 8), _host_memref(pkg, (2, 9, 4)),
                   _host_memref(pkg, (2, 3, 4)))
    with pytest.raises(pkg.HomError):
        hom.cu_seqlen("I64", _host_memref(pkg, (4, 8), 8), _host_memref(pkg, (4,), 4))
    with pytest.raises(pkg.HomError):  # cu_seqlens must have bs + 1 entries
        hom.nvteBertAttentionF16(_host_memref(pkg, (2, 128, 384)), _host_memref(pkg, (2,), 4),
                                 _host_memref(pkg, (2, 128, 128)), 0.125, 2)
    for stub in ("cutlassGemmF32", "nvteBertAttentionF32", "cutlassLayernormGemmF32"):
        hom.clear_error()
        fn = getattr(hom.lib, stub)
        args = []
        for t in fn.argtypes:
            args.append(t(0) if t is not ctypes.c_void_p else None)
        fn(*args)
        assert hom.last_error()[0] == 2, stub
    hom.clear_error()
    assert hom.launch_count() == before


def test_error_channel_clears(pkg, hom):
    hom.lib.nvteLayernormF16(0, None, 1e-5)
    code, msg = hom.last_error()
    assert code == 1 and "nvteLayernormF16" in msg
    hom.clear_error()
    assert hom.last_error() == (0, "")


def test_zero_sized_calls_are_no_ops(pkg, hom):
    before = hom.launch_count()
    hom.cutlassGemmF16(_host_memref(pkg, (1, 0, 64)), _host_memref(pkg, (1, 64, 64)), None,
                       _host_memref(pkg, (1, 0, 64)))
    assert hom.launch_count() == before


def test_tile_table_covers_the_bert_shapes(hom):
    for m, n, k, act in [(4096, 2304, 768, 0), (4096, 768, 768, 0), (4096, 3072, 768, 1),
                         (4096, 768, 3072, 0), (512, 3072, 768, 1)]:
        q = hom.gemm_query_tile(m, n, k, act)
        assert 1 <= q["row"] <= 6 and q["bn"] in (64, 128, 192, 256) and q["stages"] >= 4
    q = hom.gemm_query_tile(100, 64, 64, 0)  # unknown shape: heuristic
    assert q["bn"] in (64, 128, 192, 256) and q["stages"] >= 4
    big = hom.gemm_query_tile(16384, 4096, 1024, 1)  # large problems go to CTA pairs
    assert big["row"] == 6 and big["bn"] == 256


def test_tuned_table_round_trips_through_a_cache_file(hom, tmp_path):
    """The tuned table (the stand-in for GemmProfiler's timing cache) overrides the built-in
    choice, and what is saved is what is loaded."""
    src = tmp_path / "tuned.txt"
    # "M N K activation row [split]"; a line without the split means 1; row 9 is not a table row
    src.write_text("1000 520 264 0 2\n1000 520 264 1 5 3\n77 8 8 0 9\n")
    assert hom.gemm_tune_load(src) == 2
    q = hom.gemm_query_tile(1000, 520, 264, 0)
    assert (q["row"], q["split_k"]) == (2, 1)
    q = hom.gemm_query_tile(1000, 520, 264, 1)
    assert (q["row"], q["split_k"]) == (5, 3)
    out = tmp_path / "saved.txt"
    assert hom.gemm_tune_save(out) >= 2
    lines = {tuple(map(int, l.split())) for l in out.read_text().splitlines()}
    assert (1000, 520, 264, 0, 2, 1) in lines and (1000, 520, 264, 1, 5, 3) in lines
    assert hom.gemm_tune_load(tmp_path / "missing.txt") == -1


def test_shard_batch(pkg):
    from hands_on_mlir_b200.bert_program import shard_batch
    spans = [shard_batch(256, 8, r) for r in range(8)]
    assert spans[0] == (0, 32) and spans[-1] == (224, 256)
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        shard_batch(10, 4, 0)


def test_synthetic_inputs_do_not_depend_on_the_sharding():
    import bench
    wl = bench.WORKLOADS["bert-large"]
    ids, mask, types = bench.make_inputs(wl, 8, 0)
    ids2, mask2, _ = bench.make_inputs(wl, 4, 4)
    np.testing.assert_array_equal(ids[4:], ids2)
    np.testing.assert_array_equal(mask[4:], mask2)
    lens = mask.sum(1)
    assert ((lens >= 256) & (lens <= 512)).all()
    assert (ids[mask == 0] == 0).all() and (ids[mask == 1] >= 1000).all() and not types.any()
    idsb, maskb, _ = bench.make_inputs(bench.WORKLOADS["bert-base"], 4, 0)
    assert maskb.all() and idsb.min() >= 1000 and idsb.max() < 30522


def test_flop_model_matches_the_survey_figures(pkg):
    from hands_on_mlir_b200.bert_program import BertConfig
    base = BertConfig.base()
    assert 32 * base.gemm_flops_per_sequence(128) == 695_784_701_952
    assert 32 * base.attention_flops_per_sequence(128) == 12 * 1_610_612_736
    assert len(base.weight_names()) == 3 + 4 * 12
    assert base.weight_shape("w1_3", 128) == (1, 768, 3072)
    assert base.weight_shape("w1_3", 128, nk=True) == (1, 3072, 768)


def test_model_loader_protocol_on_cpu(pkg, hom, tmp_path):
    """The LLVM-free loader against a stub model library that touches no GPU: argNum and initFn
    run once, hoisted tensors come first, user arguments keep their slots, the result comes
    back through the last slot."""
    import subprocess
    from hands_on_mlir_b200.bert_program import ModelLibrary
    so = tmp_path / "libecho.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(so),
                    str(REPO / "tests" / "model_stub" / "cpu_echo_model.c")], check=True)
    model = ModelLibrary(so)
    assert model.init_tensor_count("forward") == -1  # nothing cached before the first call
    x = pkg.MemRef(0xABC0, (4, 8))
    for call in range(2):
        res = model.invoke("forward", [x, ctypes.c_int32(7 + call)])
        rec = ctypes.cast(res.descriptor, ctypes.POINTER(ctypes.c_int64))
        assert res.rank == 2
        assert [rec[i] for i in range(6)] == [1, 1000, 2, 1001, 3, 1002]
        assert rec[6] == 2 and rec[7] == 0xABC0 and rec[8] == 7 + call
        assert rec[9] == 1  # initFn ran exactly once
    assert model.init_tensor_count("forward") == 3
    with pytest.raises(pkg.HomError):
        model.invoke("no_such_function", [])
    model.close()
