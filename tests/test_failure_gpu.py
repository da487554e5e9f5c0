"""A wait inside a kernel that runs out must reach the host and fail the step's requests, not end as wrong tokens.

The tcgen05 product bounds every wait on a barrier; a test hook of its library (`tl_gemm_tc_test_hooks`) shortens
the bound to about a millisecond and makes the copy thread leave out its last stage of operands, so the MMA thread's
wait for that stage runs out: the block records its status code, frees its tensor memory and returns with invalid
output.  Nothing is left in flight and the GPU context stays usable.  The engine must raise `KernelError`, fail every
request (tzar-beep/Tensorline fans an exception out to all requests: tensorline/batch_engine.py:568-576), give every
page back, and serve the next request once the hook is off."""
import ctypes

import pytest
import torch

from tests.tiny import CONFIGS, PAGE_SIZE, random_tokens, write_tiny

pytestmark = pytest.mark.gpu


@pytest.fixture()
def hooks(monkeypatch):
    from tensorline_b200 import ops_gemm
    from tensorline_b200.parts import linear
    monkeypatch.setattr(linear, "TC_MIN_WEIGHT_ELEMENTS", 0)            # the tiny model's products take the tcgen05 kernel
    fn = ops_gemm.lib().tl_gemm_tc_test_hooks
    fn.argtypes = [ctypes.c_longlong, ctypes.c_int]
    fn.restype = None
    yield fn
    fn(0, 0)
    torch.cuda.synchronize()
    from tensorline_b200 import ops
    ops.device_status(torch.device("cuda"))[:1].zero_()


@pytest.mark.parametrize("graphs", [False, True])
def test_a_wait_that_runs_out_fails_the_requests_and_the_engine_goes_on(tmp_path, hooks, graphs):
    from tensorline_b200 import Engine, SamplingParams, ops
    from tensorline_b200.ops import KernelError
    folder = write_tiny("C", tmp_path / "c")
    V = CONFIGS["C"]["vocab_size"]
    prompts = [random_tokens(V, n, seed=n) for n in (9, 20)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    opts = dict(dtype="bfloat16", block_size=PAGE_SIZE["C"], num_blocks=16, max_num_seqs=4, max_model_len=64,
                cuda_graphs=graphs, overlap=graphs)
    eng = Engine(str(folder), **opts)
    launches = ops.launch_count()
    healthy = [o.token_ids for o in eng.generate(prompts, sp)]
    assert ops.launch_count() > launches
    broken = Engine(str(folder), **opts)                     # an engine of its own: graphs keep the arguments they were captured with
    reqs = [broken.add_request(p, sp) for p in prompts]
    broken.step()                                            # the prompts, still healthy
    assert all(r.num_generated == 1 for r in reqs)
    hooks(2_000_000, 1)                                      # waits give up after about a millisecond; the last stage never comes
    with pytest.raises(KernelError, match="gave up on a wait"):
        while any(not r.done for r in reqs):
            broken.step()
    assert all(r.done and isinstance(r.error, KernelError) for r in reqs)
    st = broken.stats()
    assert st["free_pages"] == st["num_pages"] and broken.cache.num_free_slots == 4
    hooks(0, 0)
    torch.cuda.synchronize()
    assert int(ops.device_status(torch.device("cuda"))[0].item()) == 0      # the word was cleared when it was raised
    again = [o.token_ids for o in eng.generate(prompts, sp)]                 # the engine (and the GPU) go on
    assert again == healthy
