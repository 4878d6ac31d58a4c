"""What the compiler made of the kernels, read from its own report (`-Xptxas -v`), without a GPU:
nothing spills, and the kernels whose design rests on two blocks sharing an SM stay within the
registers that allows. The first run compiles the kernel libraries (about a minute); later runs find
them built."""
import re

import pytest


def _entries(log):
    """[(mangled kernel name, registers, spill stores, spill loads)] of one module's report."""
    out, name = [], None
    spills = (0, 0)
    for line in log.splitlines():
        m = re.search(r"Compiling entry function '([^']+)'", line)
        if m:
            name = m.group(1)
            continue
        m = re.search(r"(\d+) bytes spill stores, (\d+) bytes spill loads", line)
        if m:
            spills = (int(m.group(1)), int(m.group(2)))
            continue
        m = re.search(r"Used (\d+) registers", line)
        if m and name:
            out.append((name, int(m.group(1)), spills[0], spills[1]))
            name = None
    return out


@pytest.fixture(scope="module")
def reports():
    from vllm_oxide_b200.csrc import build
    build.build_all(verbose=False)
    return {m: _entries(build.ptxas_log(m)) for m in build.CUDA_MODULES}


def test_no_kernel_spills(reports):
    assert all(reports[m] for m in reports), [m for m in reports if not reports[m]]
    bad = [(m, n, st, ld) for m, es in reports.items() for n, _, st, ld in es if st or ld]
    assert not bad, bad


def test_kernels_that_share_an_sm_in_pairs_keep_their_registers(reports):
    """65,536 registers per SM: two blocks of 224 threads (the few-token product: 7 warps, registers
    handed out per warp in units of 256) leave 146 per thread, two blocks of 128 (decode attention at
    head size 64, three of which share an SM) far more. The few-token product is compiled for one
    block per SM at least (`__launch_bounds__(224, 1)`), so the compiler would not object."""
    few = [(n, r) for n, r, _, _ in reports["gemm_sm100"] if "gemm_sm100_kernel" in n]
    assert few and all(r <= 144 for _, r in few), [x for x in few if x[1] > 144]
    dec64 = [(n, r) for n, r, _, _ in reports["attention_mma"] if "attn_decode_mma_kernelILi64E" in n]
    assert dec64 and all(r <= 128 for _, r in dec64), dec64
    pf = [(n, r) for n, r, _, _ in reports["attention_sm100"] if "attn_prefill_sm100_kernel" in n]
    assert pf and all(r <= 168 for _, r in pf), pf
