"""Prints a launch plan of this library's single-CTA kernel as `patina.kernel` dialect text,
and re-derives the dialect verifier's choreography rules on such text.

The reference expresses a kernel one level above PTX as text in its own MLIR dialect
(crates/patina/tests/golden/v2_gemm_pipelined.mlir:30-94, printed by crates/patina/src/emit.rs)
and checks it with C++ verifiers (mlir/lib/PatinaOps.cpp). This module closes that loop from
the other side: `kernel_text` prints the role / stage / expect_tx skeleton that one of this
library's 1-CTA tile configurations runs (load warp, MMA warp, four epilogue warps; an
S-stage ring; `full`/`empty` barriers; one accumulator barrier), in the golden file's syntax, so
that wherever the reference's `patina-opt` is built the choreography can be handed to its
verifiers. Version 0.1 of the dialect can spell less than the kernels here do
(mlir/include/patina/PatinaAttrs.td:17-24 admits `swizzle_none` only; element types are f16 in,
f32 out; one CTA), so three fields are printed as the dialect's nearest legal spelling and
listed in `SPELLING_NOTES`: the 128-byte swizzle as `swizzle_none`, bf16 / e4m3 operands as
f16, the bf16 TMA-store epilogue as the f32 `tmem_ld` + `store` pair. What the verifiers
check (byte sums, role legality, warp budget, TMEM pairing, phase order) does not depend on
those fields except through the element size, which is why byte counts are printed for the
spelled type (2 bytes), with K per stage chosen so that the bytes equal the real kernel's.

`check_text` implements, on the text, the rules the reference's verifiers enforce:
  * warp budget: sum of role warps x 32 == block            (PatinaOps.cpp:191-204)
  * expect_tx_stage bytes == sum of the bytes of the tma_load destinations that complete on
    that (pipeline, kind)                                     (PatinaOps.cpp:640-670)
  * wait_stage kinds are `empty` / `full`, `empty` only in the load role and `full` only in
    the mma role                                              (PatinaOps.cpp:790-806)
  * every tmem.alloc has exactly one tmem.dealloc             (PatinaOps.cpp:536-549)
  * the producer's loop starts at phase 1, the consumer's at phase 0
    (crates/patina/src/trace.rs:629-631)
It is host-only text processing: no device, no MLIR library.
"""
from __future__ import annotations

import re
from dataclasses import dataclass

SPELLING_NOTES = (
    "swizzle: the kernels use the 128-byte swizzle; the dialect admits swizzle_none only",
    "element type: bf16 / e4m3 operands are spelled f16 (same 2-byte width; e4m3 stages are "
    "spelled with half the K extent so that the byte counts are the kernel's)",
    "epilogue: TMEM -> registers -> swizzled shared memory -> TMA store of bf16 is spelled as "
    "the dialect's tmem_ld + store of f32",
)


@dataclass
class KernelShape:
    """What `kernel_text` prints: one CTA, tile 128 x block_n, `stages` ring stages holding
    `block_k` f16-sized elements of K each, `umma_k` elements per MMA instruction."""
    name: str = "patina_b200_gemm"
    block_n: int = 256
    block_k: int = 64            # elements per stage at 2 bytes each (128 bytes of K)
    stages: int = 4
    umma_k: int = 16
    k_advance_units: int = 2     # descriptor units between the K16 steps of a stage
    tmem_cols: int = 256
    epi_warps: int = 4


def shape_from_plan(plan, name: str = "patina_b200_gemm") -> KernelShape:
    """From a `PatinaGemmPlan` (see `lib.plan`) of a single-CTA, one-sub-tile configuration."""
    if plan.cta_group != 1 or plan.m_sub != 1:
        raise ValueError("the dialect (version 0.1) describes one CTA with one 128-row accumulator")
    # a stage holds one or more 128-byte spans of K for 128 rows of A and block_n rows of B
    spans, rest = divmod(plan.stage_bytes, (128 + plan.block_n) * 128)
    if rest or spans < 1:
        raise ValueError("unexpected stage layout")
    return KernelShape(name=name, block_n=plan.block_n, block_k=64 * spans, stages=plan.stages,
                       tmem_cols=plan.tmem_cols)


def kernel_text(k: KernelShape) -> str:
    """The kernel as dialect text, in the layout of the reference's golden file."""
    if k.block_k % k.umma_k != 0 or k.block_k % 8 != 0:
        raise ValueError("block_k must be a whole number of MMA steps and of 8-element core matrices")
    a_ty = f"!patina.tensor<f16, 128x{k.block_k}, smem, #lay>"
    b_ty = f"!patina.tensor<f16, {k.block_n}x{k.block_k}, smem, #lay>"
    tx = (128 + k.block_n) * k.block_k * 2
    cores = k.block_k // 8                       # 8-element core matrices of K per stage
    steps = k.block_k // k.umma_k
    block = 32 * (2 + k.epi_warps)
    L = []
    L.append("#lay = #patina.umma_k_major<swizzle_none>")
    L.append("")
    L.append(f"patina.kernel @{k.name}")
    L.append(f"    version = 0.1, arch = #patina.arch<sm_100a>, block = {block},")
    L.append(f"    roles = [#patina.role<load, 1>, #patina.role<mma, 1>, #patina.role<epi, {k.epi_warps}>]")
    L.append("  (%tma_a:   !patina.tma_map<f16, #lay>,")
    L.append("   %tma_b:   !patina.tma_map<f16, #lay>,")
    L.append("   %c:       !patina.ptr<f32, gmem>,")
    L.append("   %k_tiles: !patina.u32) {")
    L.append("")
    L.append(f"  %pipe = patina.pipeline.create stages = {k.stages} : !patina.pipeline<{k.stages}>")
    L.append("")
    L.append(f"  %sa = patina.smem_alloc stages = {k.stages} : {a_ty}")
    L.append(f"  %sb = patina.smem_alloc stages = {k.stages} : {b_ty}")
    L.append("")
    L.append("  %acc_done = patina.mbarrier.create arrivals = 1 : !patina.mbarrier<1>")
    L.append("")
    L.append(f"  %acc = patina.tmem.alloc cols = {k.tmem_cols} : !patina.tmem<f32, {k.tmem_cols}>")
    L.append("")
    L.append("  patina.warp_specialize {")
    L.append("")
    L.append("    patina.role load {")
    L.append("      patina.for %i = 0 to %k_tiles iter_args(%s = 0, %ph = 1) {")
    L.append("        patina.wait_stage %pipe, empty, %s, %ph")
    L.append(f"        patina.expect_tx_stage %pipe, full, %s, {tx}")
    L.append(f"        %sa_s = patina.stage_buf %sa, %s : {a_ty}")
    L.append(f"        %sb_s = patina.stage_buf %sb, %s : {b_ty}")
    L.append(f"        %i{cores}   = patina.muli %i, {cores}")
    L.append(f"        patina.tma_load %tma_a -> %sa_s, coords [0, 0, %i{cores}, 0], complete %pipe, full, %s")
    L.append(f"        patina.tma_load %tma_b -> %sb_s, coords [0, 0, %i{cores}, 0], complete %pipe, full, %s")
    L.append("        %s1, %ph1 = patina.stage_next %s, %ph of %pipe")
    L.append("        patina.yield %s1, %ph1")
    L.append("      }")
    L.append("    }")
    L.append("")
    L.append("    patina.role mma {")
    L.append("      patina.for %i = 0 to %k_tiles iter_args(%s = 0, %ph = 0) {")
    L.append("        patina.wait_stage %pipe, full, %s, %ph")
    L.append(f"        %sa_s = patina.stage_buf %sa, %s : {a_ty}")
    L.append(f"        %sb_s = patina.stage_buf %sb, %s : {b_ty}")
    L.append("        %cont = patina.nez %i")
    L.append("        %m    = patina.umma.begin %acc, %sa_s, %sb_s")
    L.append("        patina.umma.step %m, accum %cont")
    for _ in range(steps - 1):
        L.append(f"        patina.umma.advance_k %m, {k.k_advance_units}")
        L.append("        patina.umma.step %m {accum = true}")
    L.append("        patina.umma.commit %m -> %pipe, empty, %s")
    L.append("        %s1, %ph1 = patina.stage_next %s, %ph of %pipe")
    L.append("        patina.yield %s1, %ph1")
    L.append("      }")
    L.append("      patina.umma.commit %m -> %acc_done")
    L.append("    }")
    L.append("")
    L.append("    patina.role epi {")
    L.append("      patina.wait %acc_done, phase = 0")
    L.append(f"      %frag = patina.tmem_ld %acc : !patina.frag<f32, {k.tmem_cols}>")
    L.append("      patina.store %c, %frag")
    L.append("    }")
    L.append("  }")
    L.append("")
    L.append("  patina.tmem.dealloc %acc")
    L.append("}")
    return "\n".join(L) + "\n"


def normalize(text: str) -> list[str]:
    """The golden-file comparison's normalisation (crates/patina/src/testing.rs:36-58): comment
    lines dropped, trailing comments cut, trailing blanks trimmed, outer blank lines dropped."""
    out = []
    for line in text.splitlines():
        t = line.rstrip()
        if t.lstrip().startswith("//"):
            continue
        i = t.find("//")
        if i >= 0:
            t = t[:i].rstrip()
        out.append(t)
    while out and not out[0]:
        out.pop(0)
    while out and not out[-1]:
        out.pop()
    return out


_DTYPE_BYTES = {"f16": 2, "bf16": 2, "f32": 4, "f8": 1}


def _tensor_bytes(ty: str) -> int:
    m = re.search(r"!patina\.tensor<(\w+),\s*([0-9x]+),", ty)
    if not m:
        raise ValueError(f"cannot read tensor type '{ty}'")
    n = 1
    for d in m.group(2).split("x"):
        n *= int(d)
    return n * _DTYPE_BYTES[m.group(1)]


def check_text(text: str) -> list[str]:
    """Diagnostics (empty when the text passes) for the rules listed in the module docstring,
    worded like the reference's verifier messages."""
    lines = normalize(text)
    errs: list[str] = []
    joined = "\n".join(lines)
    # warp budget
    block = re.search(r"block\s*=\s*(\d+)", joined)
    roles = re.findall(r"#patina\.role<(\w+),\s*(\d+)>", joined)
    if not block or not roles:
        return ["no patina.kernel header with block and roles found"]
    warps = sum(int(w) for _, w in roles)
    if warps * 32 != int(block.group(1)):
        errs.append(f"roles require {warps} warps ({warps * 32} threads) but block = {block.group(1)}")
    # value types: smem_alloc and stage_buf results
    types: dict[str, str] = {}
    for ln in lines:
        m = re.match(r"\s*(%\w+)\s*=\s*patina\.(smem_alloc|stage_buf)\b.*:\s*(!patina\.tensor<.*>)\s*$", ln)
        if m:
            types[m.group(1)] = m.group(3)
    # role regions
    role = None
    depth_at_role = None
    depth = 0
    loads: list[tuple[str, str, str]] = []       # (pipe, kind, dst)
    expects: list[tuple[str, str, int]] = []
    for ln in lines:
        m = re.match(r"\s*patina\.role\s+(\w+)\s*\{", ln)
        if m:
            role, depth_at_role = m.group(1), depth
        m = re.match(r"\s*patina\.wait_stage\s+(%\w+),\s*(\w+),", ln)
        if m:
            kind = m.group(2)
            if kind not in ("empty", "full"):
                errs.append(f"unknown pipeline barrier kind '{kind}' (must be 'empty' or 'full')")
            else:
                need = "load" if kind == "empty" else "mma"
                if role != need:
                    errs.append(f"'patina.wait_stage' on '{kind}' barriers is only legal in a '{need}' role region")
        m = re.match(r"\s*patina\.for\b.*iter_args\(%\w+\s*=\s*\d+,\s*%\w+\s*=\s*(\d+)\)", ln)
        if m and role in ("load", "mma"):
            want = 1 if role == "load" else 0
            if int(m.group(1)) != want:
                errs.append(f"the {role} role's ring loop must start at phase {want}, not {m.group(1)}")
        m = re.match(r"\s*patina\.tma_load\s+%\w+\s*->\s*(%\w+),.*complete\s+(%\w+),\s*(\w+),", ln)
        if m:
            loads.append((m.group(2), m.group(3), m.group(1)))
        m = re.match(r"\s*patina\.expect_tx_stage\s+(%\w+),\s*(\w+),\s*%\w+,\s*(\d+)", ln)
        if m:
            expects.append((m.group(1), m.group(2), int(m.group(3))))
        depth += ln.count("{") - ln.count("}")
        if role is not None and depth <= depth_at_role:
            role = None
    for pipe, kind, nbytes in expects:
        total = 0
        for lp, lk, dst in loads:
            if lp == pipe and lk == kind:
                if dst not in types:
                    errs.append(f"cannot resolve type of tma_load destination '{dst}'")
                    continue
                total += _tensor_bytes(types[dst])
        if total != nbytes:
            errs.append(f"expect_tx_stage bytes ({nbytes}) != sum of tma_load bytes on this stage barrier ({total})")
    # TMEM pairing
    for m in re.finditer(r"(%\w+)\s*=\s*patina\.tmem\.alloc\b", joined):
        n = len(re.findall(r"patina\.tmem\.dealloc\s+" + re.escape(m.group(1)) + r"\b", joined))
        if n != 1:
            errs.append("tmem.alloc result must be consumed by exactly one patina.tmem.dealloc")
    return errs
