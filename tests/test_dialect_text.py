"""The dialect-text bridge: this library's single-CTA tile configurations printed as
`patina.kernel` text in the reference's golden syntax, and the verifier rules re-derived on that
text (warp budget, expect_tx byte sums, role legality of wait_stage, TMEM pairing, phase order).
Host-only."""
import os

import pytest

from patina_b200 import dialect_text as dt
from patina_b200 import lib as L

# the reference checkout, where there is one: PATINA_REFERENCE_ROOT, else a sibling of this repository
_REF_ROOT = os.environ.get("PATINA_REFERENCE_ROOT") or os.path.abspath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference"))
GOLDEN = os.path.join(_REF_ROOT, "crates", "patina", "tests", "golden", "v2_gemm_pipelined.mlir")


def test_every_single_cta_plan_prints_and_verifies(built_lib):
    for block_n in (256, 128, 64):
        plan = L.plan(L.IN_BF16, L.OUT_BF16, 1024, 1024, 1024, L.GemmConfig(1, block_n, 0, 0, 0))
        shape = dt.shape_from_plan(plan)
        text = dt.kernel_text(shape)
        assert dt.check_text(text) == [], text
        # the printed stage bytes are the kernel's own expect_tx count
        assert f"expect_tx_stage %pipe, full, %s, {plan.expect_tx_bytes}" in text
        assert f"stages = {plan.stages}" in text and "block = 192" in text
        # four K16 steps per 128-byte span of K in a stage
        assert text.count("patina.umma.step") == 4 * plan.stage_bytes // ((128 + block_n) * 128)
    pair = L.plan(L.IN_BF16, L.OUT_BF16, 8192, 8192, 8192)
    with pytest.raises(ValueError):
        dt.shape_from_plan(pair)                             # CTA pairs cannot be spelled in version 0.1


def test_checker_reports_what_the_reference_verifiers_report():
    good = dt.kernel_text(dt.KernelShape())
    assert dt.check_text(good) == []
    # wrong expect_tx bytes (the reference's ffi_verify.rs negative case)
    bad = good.replace("%s, 49152", "%s, 49153")
    assert any("expect_tx_stage bytes (49153) != sum of tma_load bytes on this stage barrier (49152)" in e
               for e in dt.check_text(bad))
    # misspelled barrier kind
    bad = good.replace("patina.wait_stage %pipe, empty,", "patina.wait_stage %pipe, emtpy,")
    assert any("unknown pipeline barrier kind 'emtpy'" in e for e in dt.check_text(bad))
    # consumer wait in the producer's region
    bad = good.replace("patina.wait_stage %pipe, empty,", "patina.wait_stage %pipe, full,")
    assert any("only legal in a 'mma' role region" in e for e in dt.check_text(bad))
    # warp budget
    bad = good.replace("block = 192", "block = 128")
    assert any("roles require 6 warps (192 threads) but block = 128" in e for e in dt.check_text(bad))
    # TMEM pairing
    bad = good.replace("  patina.tmem.dealloc %acc\n", "")
    assert any("exactly one patina.tmem.dealloc" in e for e in dt.check_text(bad))
    # phase convention
    bad = good.replace("iter_args(%s = 0, %ph = 1)", "iter_args(%s = 0, %ph = 0)")
    assert any("must start at phase 1" in e for e in dt.check_text(bad))


@pytest.mark.skipif(not os.path.isfile(GOLDEN), reason="reference checkout not present")
def test_reference_shape_reproduces_the_golden_text():
    """With the reference kernel's own parameters (128 x 128 tile, 32 halves of K per stage, 4
    stages, K-advance 16, 128 TMEM columns) the generator prints the reference's golden dialect
    text line for line (after the golden comparison's normalisation), and the checker accepts
    the golden file as it accepts our own text."""
    golden = open(GOLDEN).read()
    assert dt.check_text(golden) == []
    ours = dt.kernel_text(dt.KernelShape(name="tcgen05_gemm_v2", block_n=128, block_k=32, stages=4, umma_k=16,
                                         k_advance_units=16, tmem_cols=128))
    assert dt.normalize(ours) == dt.normalize(golden)
