"""The checked build (CPMCU_CHECK_BOUNDS=1: every page number a kernel takes from a page table is checked before it
is used, and every region of the arena is followed by guard words), run in a process of its own because the choice
is made when the kernel library is loaded.  It stands in for a memory checker, which cannot be run here.

A bad page number is made in a way that cannot fault: the cache's tensors hold 16 pages, the kernels are told that
it holds 10, and a page table names page 12; a kernel that followed it would still read memory of the cache."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CLEAN = r'''
import os, sys, tempfile, torch
from cpmcu_b200 import LLM
from cpmcu_b200.ops import library
from tests import configs, helpers
with tempfile.TemporaryDirectory() as tmp:
    for name, cfgd, dtype in (("b", configs.tiny_b(), "bfloat16"), ("a", configs.tiny_a(), "float32"), ("e", configs.tiny_e(), "bfloat16")):
        folder = helpers.make_folder(cfgd, os.path.join(tmp, name), 1, dtype)
        llm = LLM(folder, dtype=dtype, cuda_graph=True, max_tokens=64 * 16, chunk_length=64, max_batch=4)
        prompts = [helpers.random_ids(cfgd["vocab_size"], n, n) for n in (100, 7, 300 if name == "e" else 90)]
        res = llm.generate_batch(prompts, generation_length=8)
        assert all(len(r.tokens) == 8 for r in res)
        llm.ops.raise_on_kernel_error()                 # bounds records of every file, guard words of every region
        assert llm.storage.arena.guards and len(llm.storage.arena.guard_at) == 6
assert "checked" in library.library_path() and len(library.load().checked_files) == 5
print("CLEAN OK")
'''

BAD_PAGE = r'''
import math, torch
from cpmcu_b200.cache import Cache
from cpmcu_b200.ops.ops import Ops
from cpmcu_b200.parts.base import CacheNeeds
for dtype in (torch.bfloat16, torch.float32):
    ops = Ops(dtype, "cuda:0")
    cache = Cache([CacheNeeds(kv_heads=2, head_dim=64)], max_tokens=64 * 16, dtype=dtype, device="cuda:0", n_slots=2)
    slot = cache.open_sequence()
    cache.reserve(slot, 130)
    cache.sync()
    lane = cache.lane(0)
    ops.set_page_limit(10)                              # "the cache holds 10 pages"; its tensors hold 16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    qkv = torch.randn(130, (4 + 4) * 64, device="cuda").to(dtype)
    pos, seq, sl = i32(list(range(130))), i32([0] * 130), i32([slot])
    q = ops.rope_store(qkv, 4, 2, 64, pos, seq, sl, lane.page_table, lane.k, lane.v, None, 1.0, 0)
    ops.raise_on_bounds_error()                         # pages 0..2: fine
    lane.page_table[slot, 1] = 12                       # inside the tensors, beyond the limit the kernels were given
    out = ops.attention_generic(q[-1:].contiguous(), lane.k, lane.v, i32([129]), i32([0]), sl, lane.page_table, 2, 0.125)
    try:
        ops.raise_on_bounds_error()
        raise SystemExit("the bad page number went unnoticed")
    except RuntimeError as e:
        assert "attention_generic.cu" in str(e) and "value 12" in str(e) and "limit 10" in str(e), str(e)
    if dtype == torch.bfloat16:
        out = ops.decode_attention(q[-1:].contiguous(), lane.k, lane.v, i32([130]), sl, lane.page_table, 2, 0.125)
        try:
            ops.raise_on_bounds_error()
            raise SystemExit("the bad page number went unnoticed by the decode kernel")
        except RuntimeError as e:
            assert "attention_bf16.cu" in str(e) and "value 12" in str(e), str(e)
    ops.raise_on_bounds_error()                         # records are cleared when read
print("BAD PAGE OK")
'''


@pytest.mark.parametrize("name,script", [("clean", CLEAN), ("bad_page", BAD_PAGE)])
def test_checked_build(name, script):
    env = dict(os.environ, CPMCU_CHECK_BOUNDS="1", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    out = subprocess.run([sys.executable, "-c", script], cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-3000:] + out.stdout[-500:]
    assert out.stdout.strip().endswith("OK")
