"""Checks on the kernels' source text that need no compiler.

Every kernel is launched with programmatic dependent launch, so it may start while the kernel ahead of it still
runs, and it must call tq_grid_wait() before it reads what that kernel wrote.  Where the wait is the kernel's first
statement nothing can come before it.  A few kernels ask for static data (weights, old keys) first and wait later;
there the compiler has been seen to move loads through `const __restrict__` pointers above the wait, so those kernels
must renew the pointers they use behind the wait (tq_fresh) or read what the kernel ahead wrote only by statements
that keep their place (TMA and cp.async are volatile assembly).  This test keeps the two lists honest."""
import os
import re

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "turboquant.cpp_b200", "csrc")

# kernels whose wait is not their first statement, and how they keep their loads behind it
LATE_WAIT = {
    "attention_split_kernel": "tq_fresh",
    "attention_gqa_kernel": "tq_fresh",
    "gemv_kernel": "gemv_stage_x",            # waits and renews x inside this helper
    "qkv_gemv_rope_kernel": "gemv_stage_x",
    "router_cluster_kernel": "tq_fresh",
    "router_tiny_kernel": "tq_fresh",
    "gemm_tc_kernel": "tma_load_2d",          # what the kernel ahead wrote comes in by TMA only (volatile assembly)
}


def kernels(text):
    """(name, body) of every __global__ function of a source file."""
    out = []
    for m in re.finditer(r"__global__\s+void(?:\s+__launch_bounds__\s*\((?:[^()]|\([^()]*\))*\))?\s+(\w+)\s*\(", text):
        i = text.index("{", m.end())
        depth, j = 0, i
        while True:
            if text[j] == "{":
                depth += 1
            elif text[j] == "}":
                depth -= 1
                if depth == 0:
                    break
            j += 1
        out.append((m.group(1), text[i + 1:j]))
    return out


def first_statement(body):
    body = re.sub(r"//[^\n]*", "", body)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    return body.strip().split(";")[0].strip()


def test_every_kernel_waits_first_or_is_known_to_wait_late():
    seen_late = set()
    n = 0
    for name in sorted(os.listdir(CSRC)):
        if not name.endswith(".cu"):
            continue
        text = open(os.path.join(CSRC, name)).read()
        for kernel, body in kernels(text):
            n += 1
            assert "tq_grid_wait()" in body or "gemv_stage_x" in body, f"{name}: {kernel} never waits for the kernel ahead"
            if first_statement(body) == "tq_grid_wait()":
                continue
            assert kernel in LATE_WAIT, (f"{name}: {kernel} does something before tq_grid_wait(); list it in LATE_WAIT "
                                         f"with the way it keeps its loads behind the wait")
            assert LATE_WAIT[kernel] in body, f"{name}: {kernel} waits late but does not use {LATE_WAIT[kernel]}"
            seen_late.add(kernel)
    assert n >= 30, f"only {n} kernels found: the pattern no longer matches the sources"
    assert seen_late == set(LATE_WAIT), f"listed but not found waiting late: {sorted(set(LATE_WAIT) - seen_late)}"


def test_the_helper_that_waits_renews_its_pointer():
    text = open(os.path.join(CSRC, "gemv.cu")).read()
    i = text.index("void gemv_stage_x(")
    body = text[i:text.index("}", text.index("__syncthreads();", i))]
    assert body.index("tq_grid_wait()") < body.index("tq_fresh(x)") < body.index("xs + i")
