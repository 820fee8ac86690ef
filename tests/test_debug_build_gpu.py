"""What stands in for a memory checker (none can be run on the GPUs these tests use): guard
bands around the engine's buffers, the page tables compared with the bookkeeping, and the
debug build (MORMOT_B200_DEBUG=1), whose kernels check every index into a page table before
they use it. The failures are made on the host: a band is damaged by the test itself, a table
entry is changed by the test, and the index that the debug build refuses lies inside a table
that is larger than the kernel is told, so that nothing is read or written outside a buffer
in any build."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from mormot2_ai_b200 import Engine, Entry
from tests.conftest import ROOT, close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_guard_bands_and_page_tables_stay_whole(tiny, dtype):
    eng = Engine.from_folder(tiny.folder, dtype=dtype, max_tokens=1024, max_slots=3, guard=True,
                             prefill_chunk=48)
    assert len(eng.rt.guards.bands) >= 4
    prompts = [tiny.tokens(n, seed=60 + n) for n in (100, 3, 64)]
    slots = [eng.open() for _ in prompts]
    out = eng.step([Entry(s, p) for s, p in zip(slots, prompts)])       # three passes
    want = np.stack([tiny.reference(p)[-1] for p in prompts])
    ok, err = close(out.cpu().numpy(), want, dtype)
    assert ok, err
    for t in range(5):
        eng.step([Entry(s, [t + 1]) for s in slots])
    eng.close(slots[1])
    s = eng.open()
    eng.step([Entry(s, tiny.tokens(70, seed=3))])
    assert eng.faults() == []
    # a write outside a buffer, made here: the band says which buffer
    name, front, back = eng.rt.guards.bands[0]
    back[17] = 0
    assert eng.faults() == [f"{name} (behind)"]
    back[17] = 0x5A
    # a table entry that differs from the bookkeeping, made here
    g0 = eng.cache.tables[0]
    kept = int(g0[slots[0], 0])
    g0[slots[0], 0] = kept + 1
    found = eng.faults()
    assert len(found) == 1 and f"slot {slots[0]}, entry 0" in found[0]
    g0[slots[0], 0] = kept
    assert eng.faults() == []


DEBUG_SCRIPT = r"""
import sys
sys.path.insert(0, sys.argv[1])
import numpy as np, torch
from mormot2_ai_b200 import Engine, Entry, KernelError
from mormot2_ai_b200 import kernels as K
from mormot2_ai_b200.csrc import build
from mormot2_ai_b200.cache.storage import CacheLine
from mormot2_ai_b200.engine.batch import StepBuffers
assert build.DEBUG_BOUNDS
eng = Engine.from_folder(sys.argv[2], dtype="float32", max_tokens=512, max_slots=2)
ids = [int(t) for t in sys.argv[3].split(",")]
slot = eng.open()
out = eng.step([Entry(slot, ids[:-1])])
out = eng.step([Entry(slot, ids[-1:])])
eng.rt.check()                                   # every index was inside its table
np.save(sys.argv[4], out.cpu().numpy())
# An index outside the table row that the kernel is told of: the table has 2 rows of 8
# entries, all of them pages that exist; the kernel is told rows of 4 entries, and slot 0's
# token stands at position 5 * 64 + 2, entry 5 of a row of 4. A build without the check would
# read entry 5 (slot 1's row: a page that exists); this build records it and uses row 0.
dev = "cuda:0"
table = torch.arange(16, dtype=torch.int32, device=dev).view(2, 8).contiguous()
k = torch.zeros((16, 1, 64, 16), dtype=torch.float32, device=dev)
line = CacheLine(k, torch.zeros_like(k), table, 4, 0, 0, 1, 16)
step = StepBuffers(64, 2, torch.device(dev)).fill([(0, 5 * 64 + 2, [0], [])])
qkv = torch.ones((1, 3 * 16), dtype=torch.float32, device=dev)
K.qk_norm_rope_store(qkv, None, None, 0.0, None, 0, step, line, 1, 1, 16, True)
try:
    eng.rt.check()
    print("NOT CAUGHT")
except KernelError as e:
    print("CAUGHT:", e)
eng.rt.check()                                   # told once, then forgotten
print("DONE")
"""


def test_the_debug_build_checks_every_page_table_index(tiny_a_model, tmp_path):
    tiny = tiny_a_model
    ids = tiny.tokens(70, seed=5)
    out = str(tmp_path / "logits.npy")
    env = dict(os.environ, MORMOT_B200_DEBUG="1")
    p = subprocess.run([sys.executable, "-c", DEBUG_SCRIPT, ROOT, tiny.folder,
                        ",".join(map(str, ids)), out], capture_output=True, text=True,
                       timeout=900, env=env)
    assert p.returncode == 0, p.stderr[-3000:]
    assert "CAUGHT:" in p.stdout and "a position outside the slot's row" in p.stdout
    assert "(0, 322, 4)" in p.stdout             # slot 0, position 322, a row of 4 entries
    assert "NOT CAUGHT" not in p.stdout and p.stdout.strip().endswith("DONE")
    ok, err = close(np.load(out), tiny.reference(ids)[-1:], "float32")
    assert ok, err                                # and the debug build computes the same
