"""Source-level check of the programmatic-dependent-launch contract: a kernel that is launched
with the programmatic stream serialization attribute may start while its predecessor is still
running, so it has to call pdl_wait() (griddepcontrol.wait) before it touches global memory.
A kernel that gains the attribute without the wait would race silently; this test names it."""
import glob
import os
import re

KERNELS = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "torch-gcu_b200", "csrc", "kernels")


def _sources():
    return {os.path.basename(f): open(f).read() for f in glob.glob(os.path.join(KERNELS, "*.cu"))}


def _pdl_launched(src):
    names = set()
    for s in src.values():
        names.update(m.group(1) for m in re.finditer(r"launch_pdl\(\s*([A-Za-z_0-9]+)", s))
        names.update(m.group(1) for m in re.finditer(r"auto kernel = ([A-Za-z_0-9]+)<", s))
        if "ProgrammaticStreamSerialization" in s:
            names.update(m.group(1) for m in re.finditer(r"cudaLaunchKernelEx\(&cfg, ([A-Za-z_0-9]+)", s))
    names.discard("kernel")
    return names


def _body(src, name):
    for s in src.values():
        m = re.search(r"\n" + name + r"\(", s)
        if m:
            return s[m.start():s.index("\n}\n", m.start())]
    return None


def test_every_pdl_launched_kernel_waits_first():
    src = _sources()
    names = _pdl_launched(src)
    assert len(names) >= 10, names          # the scan itself still finds the launches
    for name in sorted(names):
        body = _body(src, name)
        assert body is not None, "definition of %s not found" % name
        assert "pdl_wait()" in body, "%s is launched with the attribute but never calls pdl_wait()" % name
        # nothing may read through a pointer before the wait: the wait comes before the first load helper
        first_wait = body.index("pdl_wait()")
        for needle in ("load_stream16(", "tma_load_", "__ldcs(", "load_index<"):
            pos = body.find(needle)
            assert pos < 0 or pos > first_wait, "%s: %s before pdl_wait()" % (name, needle)


def test_tensor_core_kernels_trigger_after_their_tmem_allocation():
    """A successor that allocates tensor memory must not be able to start before every CTA of the
    running grid holds its own columns: the trigger comes after the allocation."""
    src = _sources()
    for name in ("gemm_tc_kernel", "gemm_tc2_kernel", "gemm_splitk_kernel", "attention_decode_kernel"):
        body = _body(src, name)
        assert body is not None
        alloc = max(body.find("tmem_alloc("), body.find("tcgen05.alloc"))
        assert alloc > 0, name
        assert body.index("pdl_launch_dependents()") > alloc, name
