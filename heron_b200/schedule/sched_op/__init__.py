"""Schedule rules of the B200 kernel family.

The reference walks a TVM schedule with rules that each apply a primitive *and* register the
knobs / constraints it implies (schedule/sched_op/gpu_tensorcore_operator.py:362-414,
schedule/primitives.py:5-37).  The rules here do the second half for the hand-written kernels:
every rule declares the knobs it owns and the constraints that tie them to the SM's limits, and
when a solved point is replayed (``Task.instantiate``) reads the values back into
``ctx.kernel_knobs``, from which the kernel is launched.
"""
from ...utils import genKey
from ..constraints.primitives import EQ

ELEM_BYTES = {"float16": 2, "float32": 4, "int8": 1, "uint8": 1, "int32": 4}


class SchedOp:
    def __init__(self, name):
        self.name = name

    def perform(self, s, stage_name, ctx):
        raise NotImplementedError


def _problem(s, stage_name):
    for out in s.outputs:
        if out.op.name == stage_name:
            return out
    raise KeyError(stage_name)


def _gemm_view(out):
    """(batch, M, N, K, k_inner) of the operator's implicit GEMM."""
    p = out.op.params
    if out.op.kind in ("gemm", "scan"):
        return 1, p["M"], p["N"], p["K"], p["K"]
    if out.op.kind == "bmm":
        return p["batch"], p["M"], p["N"], p["K"], p["K"]
    if out.op.kind == "gemv":
        return 1, p["M"], 8, p["K"], p["K"]
    if out.op.kind == "conv1d_ncw":
        N, WO = out.shape[0], out.shape[2]
        ci, taps = _nchw_k_block(p["CI"], 1, p["KW"], ELEM_BYTES[p["in_dtype"]])
        return 1, N * WO, p["CO"], taps * ci, ci
    if out.op.kind == "conv3d_ncdhw":
        gran = 32 // ELEM_BYTES[p["in_dtype"]]
        ci = (p["CI"] + gran - 1) // gran * gran
        return (1, out.shape[0] * out.shape[2] * out.shape[3] * out.shape[4], p["CO"],
                p["KD"] * p["KH"] * p["KW"] * ci, ci)
    if out.op.kind == "conv1d_nwc_packed":
        return 1, out.shape[0] * out.shape[1], p["CO"], p["KW"] * p["CI"], p["CI"]
    if out.op.kind == "conv2d_nchw":
        N, HO, WO = out.shape[0], out.shape[2], out.shape[3]
        ci, taps = _nchw_k_block(p["CI"], p["KH"], p["KW"], ELEM_BYTES[p["in_dtype"]])
        return 1, N * HO * WO, p["CO"], taps * ci, ci
    N, HO, WO = out.shape[0], out.shape[1], out.shape[2]
    return 1, N * HO * WO, p["CO"], p["KH"] * p["KW"] * p["CI"], p["CI"]


def _nchw_k_block(CI, KH, KW, es):
    """(contiguous K elements per tap, taps) of the NHWC problem the library turns an NCHW conv into.
    Channels are zero-padded to 32-byte groups; with at most 16 bytes of channels and a filter row
    of 2..8 taps, a whole filter row (padded to 4 or 8 taps of 16 bytes) is one K block instead."""
    cis = 16 // es
    if CI <= cis and 2 <= KW <= 8:
        return (4 if KW <= 4 else 8) * cis, KH
    gran = 32 // es
    return (CI + gran - 1) // gran * gran, KH * KW


class tileOp(SchedOp):
    """Accumulator tile: 128 x tile_n, and the K extent of a ring stage (= TMA swizzle span)."""

    def perform(self, s, stage_name, ctx):
        km = ctx.knob_manager
        out = _problem(s, stage_name)
        p = out.op.params
        es, eo = ELEM_BYTES[p["in_dtype"]], ELEM_BYTES[p["out_dtype"]]
        _, M, N, K, k_inner = _gemm_view(out)
        conv = out.op.kind.startswith("conv")
        tile_n = genKey("P", stage_name, "n", param_name="tile_n")
        swz = genKey("P", stage_name, "k", param_name="swizzle_bytes")
        cta_group = genKey("P", stage_name, "m", param_name="cta_group")
        bn_cta = genKey("V", stage_name, "n", var_name="tile_n_per_cta")
        a_bytes = genKey("V", stage_name, "m", var_name="a_stage_bytes")
        b_bytes = genKey("V", stage_name, "n", var_name="b_stage_bytes")
        stage_bytes = genKey("V", stage_name, "k", var_name="stage_bytes")
        if km.is_building:
            step = 64 if eo == 2 else 32
            # Swizzle spans the kernel accepts for this shape: conv blocks must not straddle
            # two filter taps, so the span has to divide the channel bytes.
            spans = [sw for sw in (32, 64, 128) if not conv or (k_inner * es) % sw == 0]
            if not spans:
                raise ValueError("conv channels of %d bytes are not a multiple of 32: outside the kernels' "
                                 "documented limits" % (k_inner * es))
            if not conv and K * es < 128:
                spans = [sw for sw in spans if sw <= max(32, 1 << ((K * es - 1).bit_length()))] or [32]
            gran = step
            if conv:
                gran = max(step, min(spans) // es)
            n_cands = [n for n in range(gran, 257, gran)]
            km.define_value(tile_n, min(n_cands), max(n_cands), n_cands[-1], True)
            km.addCandidates(tile_n, n_cands)
            km.define_value(swz, min(spans), max(spans), max(spans), True)
            km.addCandidates(swz, spans)
            # 1: every CTA owns its MMAs; 2: a CTA pair shares them (256-row tiles, half of the
            # tile's B rows staged per CTA), which needs more than one 128-row tile of work.
            km.define_value(cta_group, 1, 2 if M > ctx.limits["tile_m"] else 1, 1, True)
            km.define_value(bn_cta, 8, 256, n_cands[-1])
            km.addProd([bn_cta, cta_group], tile_n)
            lim = ctx.limits["max_shared_memory_per_block"]
            km.define_value(a_bytes, 1, lim, ctx.limits["tile_m"] * max(spans))
            km.define_value(b_bytes, 1, lim, n_cands[-1] * max(spans))
            km.define_value(stage_bytes, 1, lim, (ctx.limits["tile_m"] + n_cands[-1]) * max(spans))
            km.addProd([ctx.limits["tile_m"], swz], a_bytes)
            km.addProd([bn_cta, swz], b_bytes)
            km.addSUM(stage_bytes, [a_bytes, b_bytes])
            if conv:
                # MN-major filter tiles come in whole swizzle spans of output channels.
                chunk = genKey("V", stage_name, "n", var_name="b_chunk_bytes")
                nchunk = genKey("V", stage_name, "n", var_name="b_chunks")
                km.define_value(chunk, 1, 256 * es, 256 * es)
                km.define_value(nchunk, 1, 256, 1)
                km.addProd([bn_cta, es], chunk)
                km.addProd([nchunk, swz], chunk)
        ctx.kernel_knobs["tile_n"] = km.get_val(tile_n)
        ctx.kernel_knobs["swizzle_bytes"] = km.get_val(swz)
        ctx.kernel_knobs["cta_group"] = km.get_val(cta_group)
        ctx.addSchedDesc("\n## tile 128 x %s, %s bytes of K per stage\n"
                         % (ctx.kernel_knobs["tile_n"], ctx.kernel_knobs["swizzle_bytes"]))


class pipelineOp(SchedOp):
    """Depth of the TMA -> MMA ring, swizzle spans of K per ring stage, and number of TMEM
    accumulator buffers."""

    def perform(self, s, stage_name, ctx):
        km = ctx.knob_manager
        stages = genKey("P", stage_name, "k", param_name="stages")
        acc = genKey("P", stage_name, "n", param_name="acc_stages")
        ring = genKey("V", stage_name, "k", var_name="ring_bytes")
        cols = genKey("V", stage_name, "n", var_name="tmem_columns")
        tile_n = genKey("P", stage_name, "n", param_name="tile_n")
        stage_bytes = genKey("V", stage_name, "k", var_name="stage_bytes")
        slices = genKey("P", stage_name, "k", param_name="k_slices")
        if km.is_building:
            lim = ctx.limits["max_shared_memory_per_block"]
            km.define_value(stages, 1, ctx.limits["max_stages"], 4, True)
            # swizzle spans of K behind one ring barrier: the stage, and the ring, grow with it
            km.define_value(slices, 1, 2, 1, True)
            km.define_value(acc, 1, 2, 2, True)
            km.define_value(ring, 1, lim, lim)
            km.define_value(cols, 1, ctx.limits["tmem_columns"], ctx.limits["tmem_columns"])
            km.addProd([stages, slices, stage_bytes], ring)
            km.addProd([acc, tile_n], cols)
        ctx.kernel_knobs["stages"] = km.get_val(stages)
        ctx.kernel_knobs["acc_stages"] = km.get_val(acc)
        ctx.kernel_knobs["k_slices"] = km.get_val(slices)
        ctx.addSchedDesc("## ring of %s stages of %s K spans, %s accumulator buffers\n"
                         % (ctx.kernel_knobs["stages"], ctx.kernel_knobs["k_slices"],
                            ctx.kernel_knobs["acc_stages"]))


class epilogueOp(SchedOp):
    """Accumulator write-back path and the shared-memory total it leaves for the ring."""

    def perform(self, s, stage_name, ctx):
        km = ctx.knob_manager
        out = _problem(s, stage_name)
        p = out.op.params
        eo = ELEM_BYTES[p["out_dtype"]]
        _, M, N, K, _ = _gemm_view(out)
        epi = genKey("P", stage_name, "n", param_name="epilogue")
        epi_bytes = genKey("V", stage_name, "n", var_name="epilogue_bytes")
        smem = genKey("V", stage_name, "k", var_name="shared_mem_size")
        ring = genKey("V", stage_name, "k", var_name="ring_bytes")
        if km.is_building:
            lim = ctx.limits["max_shared_memory_per_block"]
            # 1: shared-memory staging + TMA store (needs 16-byte output rows); 2: direct stores.
            modes = [1, 2] if (N * eo) % 16 == 0 else [2]
            km.define_value(epi, min(modes), max(modes), modes[0], True)
            km.addCandidates(epi, modes)
            km.define_value(epi_bytes, 0, ctx.limits["epilogue_staging_bytes"], 0)
            staging = [ctx.limits["epilogue_staging_bytes"], 0]
            for idx, mode in enumerate(modes):
                cond = (epi + "_cand%d" % idx).replace("P#", "O#")
                km.solver.primitives.append(EQ([epi_bytes, staging[mode - 1]], cond=cond))
            km.define_value(smem, 1, lim, lim)
            km.addSUM(smem, [ring, epi_bytes, ctx.limits["smem_slack_bytes"]])
            if smem not in km.mems:
                km.mems.append(smem)
        ctx.kernel_knobs["epilogue"] = km.get_val(epi)
        ctx.addSchedDesc("## epilogue mode %s\n" % ctx.kernel_knobs["epilogue"])


class convAlgoOp(SchedOp):
    """conv only: implicit GEMM with one im2col TMA per tap (1), resident filter + one padded
    input strip per tile (2), the same with the output channels on the MMA's M axis and 256
    positions on N (3), or the second with the three taps of a filter row taken by one MMA (4).
    The second exists only for stride-1 problems whose filter and two strips fit shared memory and
    whose padded width fits the 128 MMA rows, the third for fp16 problems with 64 or 128 output
    channels whose filter, strips and output tile fit, the fourth for fp16 problems with 64 output
    channels and an undilated three-tap filter row."""

    def perform(self, s, stage_name, ctx):
        km = ctx.knob_manager
        out = _problem(s, stage_name)
        if out.op.kind != "conv2d_nhwc":
            return
        p = out.op.params
        algo = genKey("P", stage_name, "m", param_name="conv_algo")
        if km.is_building:
            es, eo = ELEM_BYTES[p["in_dtype"]], ELEM_BYTES[p["out_dtype"]]
            cands = [1]
            if strip_applies(p, es, eo, ctx.limits):
                cands.append(2)
            if strip_wide_applies(p, es, eo, ctx.limits):
                cands.append(3)
            if strip_fused_applies(p, es, eo, ctx.limits):
                cands.append(4)
            km.define_value(algo, 1, cands[-1], 1, True)
            if cands != list(range(1, cands[-1] + 1)):
                km.addCandidates(algo, cands)
        ctx.kernel_knobs["conv_algo"] = km.get_val(algo)
        ctx.addSchedDesc("## conv algorithm %s\n" % ctx.kernel_knobs["conv_algo"])


def strip_applies(p, es, eo, limits):
    """The strip kernel's own feasibility rule (mirrors the library's check)."""
    sh, sw = p["stride"]
    dh, dw = p["dilation"]
    if (sh, sw) != (1, 1):
        return False
    CI, CO, KH, KW, pad = p["CI"], p["CO"], p["KH"], p["KW"], p["padding"]
    if (CI * es) % 128 or (CO * es) % 128 or CO > 256 or CO % (128 // eo) or CO % 16:
        return False
    Wp = p["W"] + 2 * pad
    if Wp > 128:
        return False
    R = 128 // Wp
    strip_rows = R + (KH - 1) * dh
    if strip_rows > 256:
        return False
    px = max(strip_rows * Wp, (KH - 1) * dh * Wp + (KW - 1) * dw + 128)
    strip_bytes = (px * 128 + 1023) // 1024 * 1024
    filt = (KH * KW * CI * CO * es + 1023) // 1024 * 1024
    return filt + 2 * (CI * es // 128) * strip_bytes + 1024 + 512 <= limits["max_shared_memory_per_block"]


def strip_fused_applies(p, es, eo, limits):
    """The fused-row form of the strip kernel (mirrors the library's check): the strip kernel's own
    rule with the exchange buffer added, fp16, 64 output channels, KW = 3, no dilation along W."""
    if p["in_dtype"] != "float16" or p["CO"] != 64 or p["KW"] != 3 or p["dilation"][1] != 1:
        return False
    shrunk = dict(limits, max_shared_memory_per_block=limits["max_shared_memory_per_block"] - 2 * 2 * 4 * 3 * 64 * 4)
    return strip_applies(p, es, eo, shrunk)


def strip_wide_applies(p, es, eo, limits):
    """The wide strip kernel's feasibility rule (mirrors the library's check): fp16, stride 1, 64 or
    128 output channels, and the filter, two input strips and one tile of output in shared memory."""
    sh, sw = p["stride"]
    dh, dw = p["dilation"]
    if (sh, sw) != (1, 1) or es != 2 or p["in_dtype"] != "float16":
        return False
    CI, CO, KH, KW, pad = p["CI"], p["CO"], p["KH"], p["KW"], p["padding"]
    if (CI * 2) % 128 or CO not in (64, 128):
        return False
    Wp = p["W"] + 2 * pad
    if Wp < 1 or Wp > 256:
        return False
    HO = (p["H"] - ((KH - 1) * dh + 1) + 2 * pad) + 1
    WO = (p["W"] - ((KW - 1) * dw + 1) + 2 * pad) + 1
    if HO <= 0 or WO <= 0:
        return False
    P = (HO - 1) * Wp + WO
    max_off = (KH - 1) * dh * Wp + (KW - 1) * dw
    filt = (KH * KW * CI * CO * 2 + 1023) // 1024 * 1024
    for cand in (256, 192, 128, 64):
        L = cand if P >= cand else (P + 15) // 16 * 16
        SR = (Wp - 1 + L + max_off + Wp - 1) // Wp
        strip_bytes = (SR * Wp * 128 + 1023) // 1024 * 1024
        smem = filt + 2 * (CI * 2 // 128) * strip_bytes + L * CO * eo + 1024 + 512
        if SR <= 256 and smem <= limits["max_shared_memory_per_block"]:
            return True
    return False


class rasterOp(SchedOp):
    """Order in which the persistent CTAs walk the tile grid."""

    def perform(self, s, stage_name, ctx):
        km = ctx.knob_manager
        raster = genKey("P", stage_name, "m", param_name="raster")
        if km.is_building:
            km.define_value(raster, 0, 1, 0, True)
        ctx.kernel_knobs["raster"] = km.get_val(raster)
        ctx.addSchedDesc("## raster %s\n" % ctx.kernel_knobs["raster"])


class splitKOp(SchedOp):
    """Whether the work items of a partly filled wave are cut along the reduction (the slices of a
    tile add their partial sums one after the other).  0 leaves the choice to the library, 1 turns
    it off.  Only 4-byte outputs can be added into."""

    def perform(self, s, stage_name, ctx):
        km = ctx.knob_manager
        out = _problem(s, stage_name)
        p = out.op.params
        es, eo = ELEM_BYTES[p["in_dtype"]], ELEM_BYTES[p["out_dtype"]]
        _, M, N, K, _ = _gemm_view(out)
        split_k = genKey("P", stage_name, "k", param_name="split_k")
        if km.is_building:
            most = 1
            if eo == 4:
                most = max(1, min(4, (K * es) // 128))  # every slice keeps at least one K block
            km.define_value(split_k, 0, most, 0, True)
        ctx.kernel_knobs["split_k"] = km.get_val(split_k)
        ctx.addSchedDesc("## split-K %s\n" % ctx.kernel_knobs["split_k"])


class balanceOp(SchedOp):
    """How work is dealt out to the persistent CTAs: whole tiles round-robin (1), or equal runs
    of (tile, K stage) units whose end tiles are shared with the neighbouring CTA pair (2).  0
    leaves the choice to the library.  Partial sums travel through the output, so only 4-byte
    outputs with 16-byte rows have the second form."""

    def perform(self, s, stage_name, ctx):
        km = ctx.knob_manager
        out = _problem(s, stage_name)
        p = out.op.params
        eo = ELEM_BYTES[p["out_dtype"]]
        _, M, N, K, _ = _gemm_view(out)
        balance = genKey("P", stage_name, "m", param_name="balance")
        if km.is_building:
            km.define_value(balance, 0, 2 if (eo == 4 and (N * eo) % 16 == 0) else 1, 0, True)
        ctx.kernel_knobs["balance"] = km.get_val(balance)
        ctx.addSchedDesc("## balance %s\n" % ctx.kernel_knobs["balance"])


class epilogueWarpsOp(SchedOp):
    """Warps that drain a CTA's accumulators: four (one per 32 TMEM lanes) or eight (two per 32
    lanes, half of a tile's column chunks each)."""

    def perform(self, s, stage_name, ctx):
        km = ctx.knob_manager
        warps = genKey("P", stage_name, "n", param_name="epi_warps")
        if km.is_building:
            km.define_value(warps, 4, 8, 4, True)
            km.addCandidates(warps, [4, 8])
        ctx.kernel_knobs["epi_warps"] = km.get_val(warps)
        ctx.addSchedDesc("## epilogue warps %s\n" % ctx.kernel_knobs["epi_warps"])


_METHODS = {
    "tileOp": tileOp,
    "pipelineOp": pipelineOp,
    "epilogueOp": epilogueOp,
    "rasterOp": rasterOp,
    "convAlgoOp": convAlgoOp,
    "splitKOp": splitKOp,
    "balanceOp": balanceOp,
    "epilogueWarpsOp": epilogueWarpsOp,
}


def get_op_methods(_type):
    """Rule table of a code-generation type (schedule/sched_op/__init__.py:12-21).  Both targets on
    the hot path launch the same kernel family, so they share one table."""
    if _type in ("GPU_TENSOR_CORE", "CPU"):
        return _METHODS
    raise ValueError("Unsupportted code gen type %s" % _type)


def sched_via_rule(_type, ctx, s):
    """Applies every rule to every output stage, recording (rule, stage) on the knob manager so
    that ``Task.instantiate`` can replay them (schedule/sched_op/__init__.py:23-30)."""
    get_op_methods(_type)
    for out in s.outputs:
        for rule in ("tileOp", "pipelineOp", "epilogueOp", "rasterOp", "convAlgoOp", "splitKOp", "balanceOp",
                     "epilogueWarpsOp"):
            ctx.addSched(rule, out.op.name, s)
