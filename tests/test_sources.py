"""Source-level twin of the reference's code-generation check (its `check` task greps compiler output for required and
forbidden instructions): here the kernels are inline PTX, so the instructions are looked up in the sources themselves."""
import os
import re

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "scalingcontrasts_b200", "csrc")


def _read(name):
    with open(os.path.join(ROOT, name)) as handle:
        return handle.read()


def _code_only(text):
    return "\n".join(line.split("//")[0] for line in text.splitlines())


def test_blackwell_instructions_are_where_they_should_be():
    common, forward, backward, collectives = (_read(n) for n in ("common.cuh", "loss_fwd.cu", "loss_bwd.cu", "collectives.cu"))
    for needle in ("tcgen05.mma.cta_group::1.kind::f16", "tcgen05.alloc", "tcgen05.commit", "tcgen05.ld.sync.aligned.32x32b",
                   "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes", "mbarrier.try_wait.parity"):
        assert needle in common, needle
    assert "umma_bf16(" in forward and "umma_bf16(" in backward
    assert "tcgen05.st.sync.aligned" in forward and "cp.async.bulk.tensor.3d.global.shared::cta" in forward
    assert "__ffma2_rn(" in common and "elect.sync" in common  # packed float32 math, elected-lane issue
    assert "red.global.add.v4.f32" in backward
    for needle in ("multimem.ld_reduce.relaxed.sys.global.add.v4.f32", "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2",
                   "multimem.st.relaxed.sys.global.v4.f32", "multimem.red.release.sys.global.add.u32"):
        assert needle in collectives, needle


def test_legacy_and_closed_constructs_are_absent():
    for name in os.listdir(ROOT):
        if not name.endswith((".cu", ".cuh", ".cpp", ".h")):
            continue
        code = _code_only(_read(name))
        assert "wgmma" not in code and "mma.sync" not in code and "wmma" not in code, name
        assert "::".join(("multicast", "cluster")) not in code, name  # no load may carry the cluster-multicast qualifier
        assert not re.search(r"__trap\s*\(|(?<!static_)\bassert\s*\(", code), name
        assert "cudaMalloc(" not in code and "cudaFree(" not in code.replace("cudaFree(nullptr)", ""), name


def test_every_device_wait_is_bounded():
    """No `while`/`for(;;)` spin in device code without a budget: the wait helpers are the only loops on flags."""
    common, collectives = _read("common.cuh"), _read("collectives.cu")
    assert "budget_ns" in common and "budget_ns" in collectives
    # the two mbarrier waits (polling back to back, and sleeping between polls) and the collectives' flag wait
    assert common.count("for (;;)") == 2 and collectives.count("for (;;)") == 1
    for text in (common, collectives):
        for loop in re.finditer(r"for \(;;\) \{", text):
            body = text[loop.end():loop.end() + 900]
            assert "budget_ns" in body, "a spin loop without a budget"
