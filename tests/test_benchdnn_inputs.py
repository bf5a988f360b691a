"""Matmul problems written in benchdnn's input syntax (tests/benchdnn_matmul.py).

On the CPU: the expansion rules; the C restatement against the live reference
on this repository's input file and, where the reference checkout is present,
on the reference's own matmul input files (every 2D problem the driver can
express), together with the accept / reject decision of this library's
primitive-descriptor creation.  On the GPU: every problem of this repository's
input file through every implementation that accepts it."""
import os

import numpy as np
import pytest

import benchdnn_matmul as B
from onednn_b200 import workloads as W
from oracle import oracle as O
from oracle.refdir import reference_dir

HERE = os.path.dirname(os.path.abspath(__file__))
OWN = os.path.join(HERE, "benchdnn_inputs", "matmul_quantized")


def test_expansion_multiplies_comma_lists_and_follows_batch_files(tmp_path):
    (tmp_path / "shapes").write_text("# two shapes\n4x8:8x16\n2x3:3x5_n\"named\"\n")
    (tmp_path / "main").write_text(
        "--reset\n--dt=u8:s8:s32,s8:s8:f32 --wtag=ab,ba\n"
        "--attr-zero-points=src:common:1+wei:common:-1, \\\n"
        "                   src:per_dim_1\n"
        "--batch=shapes\n"
        "--reset --skip-impl=ref\n"
        "--attr-post-ops=sum+relu\n"
        "6x4:4x2\n")
    got = list(B.expand(str(tmp_path / "main")))
    assert len(got) == 2 * 2 * 2 * 2 + 1
    first, desc = got[0]
    assert desc == "4x8:8x16" and first["dt"] == "u8:s8:s32" and first["wtag"] == "ab"
    assert first["attr-zero-points"] == "src:common:1+wei:common:-1"
    assert {s["attr-zero-points"] for s, _ in got[:-1]} == {"src:common:1+wei:common:-1", "src:per_dim_1"}
    last, desc = got[-1]
    assert desc == "6x4:4x2" and last["dt"] == "f32" and last["attr-zero-points"] == ""
    assert last["attr-post-ops"] == "sum+relu"
    assert B.command_line(last, desc) == "--matmul --attr-post-ops=sum+relu 6x4:4x2"
    assert got[8][1] == '2x3:3x5_n"named"'  # the product is walked per descriptor
    p, _ = B.build(got[8][0], got[8][1])
    assert (p.M, p.K, p.N, p.name) == (2, 3, 5, "named")


def test_policy_names_give_the_masks_benchdnn_gives_a_matmul():
    s = dict(B.DEFAULTS, _unknown=[])
    s.update({"dt": "bf16:s4:bf16", "attr-fpmath": "bf16:true",
              "attr-scales": "wei:per_ocic:f16:32x1", "attr-zero-points": "wei:per_oc:u8",
              "attr-post-ops": "add:f32:per_oc+mul:s8:per_dim_0+sub:f32:per_tensor+max:f32"})
    p, _ = B.build(s, "4x64:64x32")
    assert p.quant["wei_scale"].mask == 3 and p.quant["wei_scale"].groups == (32, 1)
    assert p.quant["wei_scale"].data.shape == (2, 32) and p.quant["wei_scale"].dt == W.F16
    assert p.quant["wei_zp"].mask == 2 and p.quant["wei_zp"].data.shape == (1, 32)
    assert [po.src1.dims for po in p.post_ops] == [(1, 32), (4, 1), (4, 32), (1, 1)]
    assert p.apply_to_int and p.fpmath == 1
    s.update({"dt": "u8:s8:s8", "attr-fpmath": "", "attr-scales": "src:per_dim_0+dst:common:4",
              "attr-zero-points": "src:per_dim_1+dst:per_dim_1", "attr-post-ops": "", "runtime_dims_masks": "1:0"})
    p, opts = B.build(s, "4x64:64x32")
    assert p.quant["src_scale"].mask == 1 and p.quant["src_zp"].mask == 2 and p.quant["dst_zp"].mask == 2
    assert float(p.quant["dst_scale"].data[0, 0]) == 4.0 and opts["runtime_m"]
    _, opts = B.build(dict(s, runtime_dims_masks="3:1"), "4x64:64x32")
    assert opts["runtime_m"] == (3, 1)
    sp, so = B.build(dict(s, strides="80x1::40x1"), "4x64:64x32")
    assert sp.src.strides == (80, 1) and sp.src.data.size == 3 * 80 + 64 and so["dst_ld"] == 40 and so["dense"].src.strides == (64, 1)
    for bad in ({"runtime_dims_masks": "4:1"}, {"strides": "8x1::"}, {"strides": "::1x4"}, {"attr-post-ops": "dw:k3s1p1"},
                {"dt": "f64"}, {"dtag": "ba"}):
        with pytest.raises(B.Skip):
            B.build(dict(s, **bad), "4x64:64x32")
    with pytest.raises(B.Skip, match="batched descriptor"):  # those go through build_batched
        B.build(s, "3x4x64:3x64x32")


def test_batched_descriptors_broadcast_and_follow_their_tags(host_engine):
    s = dict(B.DEFAULTS, _unknown=[])
    s.update({"dt": "u8:s8:s32", "stag": "acb", "wtag": "abc", "dtag": "bac", "bia-dt": "f32", "bia_mask": "5",
              "attr-post-ops": "add:s32:per_dim_0"})
    bp = B.build_batched(s, "2x3x5:1x5x4")
    assert bp.ddims == (2, 3, 4) and len(bp.mats) == 2
    storage, strides, dt, dims = bp.tensors["src"]
    assert dims == (2, 3, 5) and strides == (15, 1, 3)  # acb: the K index moves 3 elements, M is innermost
    src = np.lib.stride_tricks.as_strided(storage, dims, tuple(st * storage.itemsize for st in strides))
    wei = bp.tensors["wei"][0].reshape(1, 5, 4)
    bias = bp.tensors["bias"][0].reshape(2, 1, 4)
    add = bp.post_ops[0].src1.data.reshape(2, 1, 1)
    want = np.einsum("bmk,bkn->bmn", src.astype(np.int64), np.broadcast_to(wei, (2, 5, 4)).astype(np.int64))
    want = want + bias.astype(np.int64) + add.astype(np.int64)
    for idx, p in bp.mats:
        assert np.array_equal(p.src.data, src[idx]) and np.array_equal(p.wei.data, wei[0])
        assert np.array_equal(O.run_port(p).astype(np.int64), want[idx])
    _, impl, pd = B.run_batched(bp, host_engine, None)
    assert impl == "cuda:tcgen05:int8" or impl.startswith("cuda:ref")
    # a parameter that varies along the batch is outside the library's batched path
    with pytest.raises(B.Skip):
        B.build_batched(dict(s, **{"attr-scales": "wei:per_tensor"}), "2x3x5:2x5x4")


def _pin(path, host_engine, max_macs, known_stricter=()):
    """Every buildable problem of the file: restatement == live reference bit
    for bit, and this library creates a primitive descriptor exactly where
    the reference does (apart from `known_stricter` scale strings)."""
    from onednn_b200 import api
    from onednn_b200.runner import Prepared
    ran = rejected = 0
    for settings, desc in B.expand(path):
        try:
            p, opts = B.build(settings, desc, max_macs=max_macs)
        except B.Skip:
            continue
        line = B.command_line(settings, desc)
        try:
            want, impl, _ = O.run_ref(p, pin_ref=True)
        except RuntimeError:
            want = None
        try:
            Prepared(p, host_engine, None, opts["user_scratchpad"], opts["runtime_m"], opts["dst_ld"])
            mine = True
        except api.error as e:
            assert e.status == api.unimplemented, line
            mine = False
        if settings["attr-scales"] in known_stricter:
            assert not mine, line
            continue
        assert mine == (want is not None), "accepted by %s only: %s" % ("this library" if mine else "the reference", line)
        if want is None:
            rejected += 1
            continue
        got = O.run_port(p)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), line
        ran += 1
    return ran, rejected


def test_own_input_file_restatement_matches_the_live_reference(host_engine):
    if not O.ref_available():
        pytest.skip("reference library not built")
    ran, rejected = _pin(OWN, host_engine, 300000, known_stricter=("dst:per_oc",))
    assert ran > 2000 and rejected > 0  # a sum zero-point with a float dst is refused by both


@pytest.mark.parametrize("name,max_macs,least", [
    ("test_matmul_all", 300000, 20000), ("test_matmul_ci", 300000, 100), ("harness_matmul_strides", 300000, 150),
    ("harness_matmul_precomp_reductions", 3000000, 20), ("harness_matmul_regression", 300000, 30)])
def test_reference_input_files_restatement_matches_the_live_reference(host_engine, name, max_macs, least):
    ref = reference_dir()
    if ref is None or not O.ref_available():
        pytest.skip("reference checkout or library not present")
    path = os.path.join(ref, "tests", "benchdnn", "inputs", "matmul", name)
    ran, _ = _pin(path, host_engine, max_macs)
    assert ran >= least


@pytest.mark.parametrize("name,least", [("harness_matmul_grouped_2dby3d", 300)])
def test_reference_grouped_inputs_restatement_matches_the_live_reference(host_engine, name, least):
    """Grouped (MoE) problems of the reference's own harness: `--grouped=0:G:sizes MxK:GxKxN` with
    row-wise / K-grouped src scales, per-(expert, column) / K-grouped weight scales and zero-points,
    [G, N] bias, eltwise and per-row binary post-ops.  Wherever the reference accepts a problem the
    restatement equals it bit for bit and this library creates a primitive descriptor too."""
    from onednn_b200 import api
    from onednn_b200.runner import Prepared
    ref = reference_dir()
    if ref is None or not O.ref_available():
        pytest.skip("reference checkout or library not present")
    ran = 0
    for settings, desc in B.expand(os.path.join(ref, "tests", "benchdnn", "inputs", "matmul", name)):
        if not settings["grouped"]:
            continue
        try:
            p = B.build_grouped(settings, desc, max_macs=3000000)
        except B.Skip:
            continue
        line = B.command_line(settings, desc)
        try:
            want, _, _ = O.run_ref(p, pin_ref=True)
        except RuntimeError:
            continue
        assert np.array_equal(O.run_port(p).view(np.uint8), want.view(np.uint8)), line
        try:
            Prepared(p, host_engine)
        except api.error as e:
            raise AssertionError("accepted by the reference only (%s): %s" % (e, line))
        ran += 1
    assert ran >= least


@pytest.mark.gpu
def test_own_input_file_through_every_implementation(gpu):
    eng, strm = gpu
    rep = B.run_file(OWN, eng, strm, all_impls=True)
    assert not rep["failures"], rep["failures"][:5]
    assert set(rep["reasons"]) <= {"unimplemented"}, rep["reasons"]
    assert rep["PASSED"] > 4500 and rep["SKIPPED"] < rep["PASSED"] // 4, rep
    for impl in ("cuda:tcgen05:int8", "cuda:tcgen05:fp8", "cuda:tcgen05:woq4", "cuda:woq:skinny", "cuda:tcgen05:woq8",
                 "cuda:ref_int8:any", "cuda:ref:any"):
        assert rep["impls"].get(impl, 0) >= 20, (impl, rep["impls"])


@pytest.mark.parametrize("name,least", [("test_reorder_ci", 2000), ("test_reorder_all", 2500), ("harness_reorder_scales", 700),
                                        ("harness_reorder_saturation", 120), ("harness_reorder_decompression", 500),
                                        ("test_reorder_int4", 80)])
def test_reference_reorder_inputs_restatement_matches_the_live_reference(host_engine, name, least):
    """The reference's reorder input files (tests/benchdnn_reorder.py reads their syntax): every
    plain-layout problem the reference library accepts must give the restatement's bits, and this
    library must create a reorder primitive descriptor for it too."""
    import benchdnn_reorder as R
    from onednn_b200 import api
    ref = reference_dir()
    if ref is None or not O.ref_available():
        pytest.skip("reference checkout or library not present")
    ran = 0
    for settings, desc in R.expand(os.path.join(ref, "tests", "benchdnn", "inputs", "reorder", name)):
        try:
            ro = R.build(settings, desc)
        except R.Skip:
            continue
        if int(np.prod(ro.src.dims)) > 200000:
            continue
        try:
            want, _ = O.run_ref_reorder(ro)
        except RuntimeError:
            continue
        line = "%s %s" % ({k: v for k, v in settings.items() if v != R.DEFAULTS.get(k)}, desc)
        got = O.run_port_reorder(ro)
        assert np.array_equal(np.asarray(got).view(np.uint8), np.asarray(want).view(np.uint8)), line
        try:
            R.primitive_desc(ro, host_engine)
        except api.error as e:
            raise AssertionError("accepted by the reference only (%s): %s" % (e, line))
        ran += 1
    assert ran >= least


def test_reorder_tags_follow_benchdnn():
    import benchdnn_reorder as R
    assert R.tag_order("abx", 4) == (0, 1, 2, 3) and R.tag_order("axb", 4) == (0, 2, 3, 1)
    assert R.tag_order("xba", 4) == (2, 3, 1, 0) and R.tag_order("xba", 2) == (1, 0) and R.tag_order("axb", 2) == (0, 1)
    assert R.tag_order("adbc", 4) == (0, 3, 1, 2)
    with pytest.raises(R.Skip):
        R.tag_order("aBx16b", 4)
    s = dict(R.DEFAULTS, _unknown=[])
    s.update({"sdt": "f32", "ddt": "s8", "dtag": "axb", "attr-scales": "src:per_dim_1+dst:common:2", "attr-post-ops": "sum:0.5"})
    ro = R.build(s, "2x16x3x4")
    assert ro.dst_strides == (192, 1, 64, 16) and ro.quant["src_scale"].data.shape == (1, 16, 1, 1) and ro.beta == 0.5
    assert ro.dst_init is not None and ro.dst_init.size == 2 * 16 * 3 * 4


def test_batched_problems_match_the_live_reference_matrix_by_matrix():
    """The batched problems of this repository's input file on the reference library itself (one
    batched primitive: oracle.run_ref_nd) against the 2D restatement applied to every matrix of
    the batch: the broadcast of size-1 batch dims, bias and binary operands along any dims, masks
    that skip the batch dims and the layout of prelu weights are the reference's own."""
    if not O.ref_available():
        pytest.skip("reference library not built")
    ran = 0
    for settings, desc in B.expand(OWN):
        try:
            B.build(settings, desc)
            continue
        except B.Skip as e:
            if str(e) != "batched descriptor":
                continue
        bp = B.build_batched(settings, desc)
        fpmath, apply_to_int = bp.fpmath, bp.apply_to_int
        if bp.tensors["src"][2] in (W.S8, W.U8):  # the reference's generic int8 kernel refuses an fpmath setting
            fpmath, apply_to_int = 0, False
        line = B.command_line(settings, desc)
        got, impl = O.run_ref_nd(bp.tensors["src"], bp.tensors["wei"], bp.tensors.get("bias"), bp.ddims, bp.ddt,
                                 bp.dst_strides, bp.quant, bp.post_ops, bp.dst_init, apply_to_int, fpmath)
        assert impl.startswith("ref"), (impl, line)
        full = B._gather(np.asarray(got), bp.ddims, bp.dst_strides)
        for idx, p in bp.mats:
            want = O.run_port(p)
            assert np.array_equal(np.ascontiguousarray(full[idx]).view(np.uint8), want.view(np.uint8)), (line, idx)
        ran += 1
    assert ran > 1500


@pytest.mark.parametrize("name,least", [("test_matmul_all", 4000), ("test_matmul_multidims", 400)])
def test_reference_batched_inputs_match_the_live_reference_matrix_by_matrix(name, least):
    """The same check on the batched descriptors of the reference's own input files (three to six
    dims, broadcast batch dims, permuted tags, bias masks, binary operands along any dims)."""
    import re
    ref = reference_dir()
    if ref is None or not O.ref_available():
        pytest.skip("reference checkout or library not present")
    ran = 0
    for settings, desc in B.expand(os.path.join(ref, "tests", "benchdnn", "inputs", "matmul", name)):
        m = re.fullmatch(r"([0-9x]+):([0-9x]+).*", desc)
        if m is None or m.group(1).count("x") < 2:
            continue
        macs = int(np.prod([int(x) for x in m.group(1).split("x")])) * int(m.group(2).split("x")[-1])
        if macs > 300000:
            continue
        try:
            bp = B.build_batched(settings, desc)
        except B.Skip:
            continue
        try:
            got, impl = O.run_ref_nd(bp.tensors["src"], bp.tensors["wei"], bp.tensors.get("bias"), bp.ddims, bp.ddt,
                                     bp.dst_strides, bp.quant, bp.post_ops, bp.dst_init, bp.apply_to_int, bp.fpmath)
        except RuntimeError:
            continue
        full = B._gather(np.asarray(got), bp.ddims, bp.dst_strides)
        for idx, p in bp.mats:
            assert np.array_equal(np.ascontiguousarray(full[idx]).view(np.uint8), O.run_port(p).view(np.uint8)), \
                (B.command_line(settings, desc), idx)
        ran += 1
    assert ran >= least
