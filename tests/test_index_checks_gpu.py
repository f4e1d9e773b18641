"""The kernels' index checks (builds with TQ_DEBUG_INDEX=1): a kernel that is handed an index outside its tensor
records it, goes to valid memory instead, runs to its end, and the host raises when it looks.

The checks run in a process of their own whose kernel libraries are all the checked builds.  Before it hands a
kernel a bad index, the script makes sure that the library it is about to call really is a checked build (its
fault reader says so); in a release build these inputs would be read as they are, so nothing is launched then.
"""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

SCRIPT = r'''
import ctypes, math, os, sys, tempfile
import numpy as np, torch
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import turboquant_cpp_b200 as tq
from turboquant_cpp_b200.csrc import build
from turboquant_cpp_b200.kernels import attention as KA, elementwise as KE, moe as KM
from conftest import TINY_A

assert build.DEBUG_INDEX, "this process was to load the checked builds"
DEV = "cuda:0"
i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def checked(name):
    """The library is a checked build (only then may it be handed a bad index)."""
    rec = (ctypes.c_int * 4)()
    assert build.load_kernel(name).tq_index_fault_read(rec) == 1, f"{name} is not a checked build"


def faults_after(fn):
    fn()
    torch.cuda.synchronize()                  # no trap, no fault: the kernel ran to its end
    return build.index_faults()


# 1. a page table that names a page outside the cache, and one whose page was given back (-1)
checked("attention")
nh, nkv, hd, page, n_pages, T = 4, 2, 64, 64, 8, 2
q = torch.randn((T, nh, hd), device=DEV)
cache = torch.randn((n_pages, 2, nkv, page, hd), device=DEV)
out = torch.empty((T, nh * hd), device=DEV)
partial = torch.empty(T * nh * 3 * (hd + 2), device=DEV)
args = lambda table: (q, cache, i32([100, 70]), i32([0, 1]), i32(table), page, 0, 1 / math.sqrt(hd), out, nh, nkv, hd)
f = faults_after(lambda: KA.attention_split(*args([[1, 1000000], [2, 3]]), 3, partial))
assert len(f) == 1 and "page id" in f[0] and "1000000 is not in 0..7" in f[0], f
f = faults_after(lambda: KA.attention(*args([[1, 2], [-1, 3]])))
assert len(f) == 1 and "page id" in f[0] and "-1 is not in 0..7" in f[0], f
f = faults_after(lambda: KA.attention_split(*args([[1, 2], [4, 3]]), 3, partial))
assert f == [], f                             # the record was cleared, and a good table leaves none
want = torch.empty_like(out)
KA.attention(*args([[1, 2], [4, 3]])[:8], want, nh, nkv, hd)
assert (out - want).abs().max().item() < 1e-5
# a token whose sequence index is outside the batch, and a position beyond the table's width
f = faults_after(lambda: KA.attention(q, cache, i32([100, 70]), i32([0, 5]), i32([[1, 2], [4, 3]]), page, 0, 0.1, out, nh, nkv, hd))
assert len(f) == 1 and "sequence index" in f[0] and "5 is not in 0..1" in f[0], f
f = faults_after(lambda: KA.attention(q, cache, i32([200, 70]), i32([0, 1]), i32([[1, 2], [4, 3]]), page, 0, 0.1, out, nh, nkv, hd))
assert len(f) == 1 and "position beyond the page table" in f[0], f

# 2. a token id outside the vocabulary
checked("elementwise")
table = torch.randn((50, 32), device=DEV)
x = torch.empty((3, 32), device=DEV)
f = faults_after(lambda: KE.embed_rows(i32([4, 55, -2]), table, x))
assert len(f) == 1 and "token id" in f[0] and ("55 is not in 0..49" in f[0] or "-2 is not in 0..49" in f[0]), f
assert torch.equal(x[0], table[4]) and torch.equal(x[1], table[0])       # the bad ones went to row 0

# 3. an expert id outside the layer's experts
checked("moe")
layout = KM.ExpertLayout(6, 4, 16, DEV)
f = faults_after(lambda: KM.moe_align(i32([[0, 3], [7, 1], [2, 2]]), layout))
assert len(f) == 1 and "expert id" in f[0] and "7 is not in 0..3" in f[0], f
assert int(layout.counts.sum()) == 6          # the bad pair was counted with expert 0: every row still has a place

# 4. through the engine: a sequence whose page list was damaged on the host
with tempfile.TemporaryDirectory() as d:
    tq.write_random_folder(d, TINY_A, seed=0)
    eng = tq.Engine(tq.load_model(d, "float32", DEV), max_tokens=512, use_graphs=False)
    seq = eng.open()
    eng.step([tq.StepEntry(seq, list(range(70)), [])])
    eng.check_kernels()
    good = seq.pages[0][0]
    seq.pages[0][0] = 4096                    # what a fault in the allocator would look like
    eng.step([tq.StepEntry(seq, [5], [0])])
    try:
        eng.check_kernels()
    except tq.kernels._call.KernelError as e:
        assert "page id" in str(e) and "4096" in str(e), str(e)
    else:
        raise AssertionError("the engine did not notice the bad page id")
    seq.pages[0][0] = good
    eng.step([tq.StepEntry(seq, [6], [0])])
    eng.check_kernels()                       # and is usable afterwards
    eng.close(seq)
print("index checks ok")
'''


def test_checked_builds_record_bad_indices_and_go_on():
    env = dict(os.environ, TQ_DEBUG_INDEX="1")
    r = subprocess.run([sys.executable, "-c", f"ROOT = {ROOT!r}\n" + SCRIPT], capture_output=True, text=True,
                       timeout=900, env=env)
    assert r.returncode == 0 and "index checks ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_release_builds_keep_no_record():
    from turboquant_cpp_b200.csrc import build
    if build.DEBUG_INDEX:
        pytest.skip("this process runs the checked builds")
    import ctypes
    rec = (ctypes.c_int * 4)()
    assert build.load_kernel("elementwise").tq_index_fault_read(rec) == 0 and build.index_faults() == []
