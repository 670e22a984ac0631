"""What the engine does when something goes wrong, with every failure made on the host or by a wait
that is allowed to run out: nothing here faults, traps or hangs the device."""
import pytest
import torch

import plain_llama
import replay_util as ru
from tiny_configs import CONFIGS, make_model_folder

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {n: make_model_folder(root, n) for n in ("A", "C")}


def test_a_bounded_wait_that_runs_out_is_reported_and_the_engine_goes_on(folders):
    """A kernel waits on an mbarrier at which nothing arrives, with a small limit: it gives up, the status
    word reads "wait ran out", the step function turns that into an error, and the next step runs."""
    from llm_steadyinfer_b200.csrc import ops
    from llm_steadyinfer_b200.engine.replay import Replayer
    from llm_steadyinfer_b200.engine.step import STATUS_TEXT, StepError
    rp = Replayer(folders["A"], torch.float32, max_tokens=128)
    runner = rp.runner
    toks = ru.random_tokens(CONFIGS["A"][0]["vocab_size"], 20, 3)
    before = rp.run_step([{"id": "r", "tokens": toks, "want": [19]}], ["r"]).clone()
    gave_up = torch.zeros(1, dtype=torch.int32, device="cuda")
    for limit in (1, 64, 4096):
        gave_up.zero_()
        ops.selftest_wait_runs_out(runner.status, limit, gave_up)
        with pytest.raises(StepError) as e:
            runner.check_status()
        assert "status 4" in str(e.value) and STATUS_TEXT[4] in str(e.value)
        assert int(gave_up.item()) == 1
        assert int(runner.status.item()) == 0, "the word is cleared once it has been reported"
    with pytest.raises(ops.KernelError):
        ops.selftest_wait_runs_out(runner.status, 0)
    after = rp.run_step([{"id": "r", "tokens": toks, "want": [19]}], ["r"])
    assert torch.equal(before, after), "the context is as usable as before"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_failed_recording_runs_the_shape_directly_from_then_on(folders, dtype):
    """The recording of a decode step into a CUDA graph fails (by a flag on the host): the step's tokens are
    there all the same, that batch shape is marked and runs directly, other shapes are still recorded."""
    from llm_steadyinfer_b200 import LLM, SamplingParams
    name = "A" if dtype == "float32" else "C"
    cfg, w = plain_llama.read_model_folder(folders[name])
    V = CONFIGS[name][0]["vocab_size"]
    prompts = [ru.random_tokens(V, n, 70 + i) for i, n in enumerate([12, 30, 5])]

    def run(fail):
        llm = LLM(folders[name], dtype=dtype, max_batch=4, max_seq_len=128, max_gen_len=24, block_size=16)
        llm.runner.fail_next_capture = fail
        outs = llm.generate(prompts, [SamplingParams(ignore_eos=True, max_tokens=n) for n in (24, 10, 17)])
        return llm, [o.token_ids for o in outs]

    good_llm, good = run(False)
    llm, got = run(True)
    assert got == good
    if dtype == "float32":
        assert got == [plain_llama.generate(cfg, w, p, n) for p, n in zip(prompts, (24, 10, 17))]
    assert not good_llm.runner.capture_failed
    failed = llm.runner.capture_failed
    assert len(failed) == 1 and "injected" in next(iter(failed.values()))
    assert next(iter(failed)) not in llm.runner._graphs
    # three requests end at different times: batches of 3, 2 and 1 fall into buckets 4, 2 and 1
    assert len(llm.runner._graphs) >= 1, "the shapes whose recording did not fail are replayed from graphs"
    assert not llm.runner.fail_next_capture


def test_a_store_into_a_shared_page_is_refused_before_anything_runs(folders):
    """A hand-made second holder of a request's page: a step that would store keys there raises, a step that
    stores behind it is fine."""
    from llm_steadyinfer_b200.csrc import ops
    from llm_steadyinfer_b200.engine.replay import Replayer
    from llm_steadyinfer_b200.engine.step import StepEntry, StepError
    rp = Replayer(folders["A"], torch.float32, max_tokens=256, page_size=16)
    runner, mgr = rp.runner, rp.runner.manager
    toks = ru.random_tokens(CONFIGS["A"][0]["vocab_size"], 60, 4)
    runner.step([StepEntry("r", toks[:20], [])])                  # pages 0 and 1, the second one part full
    pool = mgr.groups[0].pool
    page = mgr.table(0, "r")[1]
    pool.retain(page)                                             # as if a second request had mounted it
    launches = ops.launch_count()
    with pytest.raises(StepError) as e:
        runner.step([StepEntry("r", toks[20:24], [3])])
    assert "shared" in str(e.value) and f"page {page}" in str(e.value) and "20..23" in str(e.value)
    assert ops.launch_count() == launches, "nothing was launched"
    assert mgr.length("r") == 20
    pool.release(page)
    first = runner.step([StepEntry("r", toks[20:40], [19])]).clone()     # fills page 1, goes on into page 2
    pool.retain(page)
    out = runner.step([StepEntry("r", toks[40:44], [3])])                # page 2 only: the shared page is read
    assert out.shape[0] == 1 and torch.isfinite(out).all() and torch.isfinite(first).all()
    runner.check_status()
    pool.release(page)
    runner.finish("r")
    mgr.check_invariant()


def test_a_schedule_that_stalls_ends_with_an_error_not_a_loop(folders):
    """If the scheduler ever found nothing to run while requests are unfinished, ``generate`` would loop for
    ever; the entry point counts such steps and, after a few, aborts the requests and raises. The stall is made
    on the host: a scheduler whose ``schedule`` returns nothing."""
    from llm_steadyinfer_b200 import LLM, SamplingParams
    llm = LLM(folders["A"], dtype="float32", max_batch=2, max_seq_len=64, max_gen_len=4, block_size=16)
    prompt = ru.random_tokens(CONFIGS["A"][0]["vocab_size"], 5, 77)
    want = llm.generate([prompt], SamplingParams(ignore_eos=True))[0].token_ids
    real = llm.scheduler.schedule
    llm.scheduler.schedule = lambda: []
    rid = llm.add_request(prompt, SamplingParams(ignore_eos=True))
    with pytest.raises(RuntimeError) as e:
        for _ in range(100):
            llm.step()
    assert "nothing to run" in str(e.value)
    assert llm.all_finished()
    assert [(s.id, s.finish_reason) for s in llm.get_finished()][-1] == (rid, "aborted")
    llm.runner.manager.check_invariant()
    llm.scheduler.schedule = real
    assert llm.generate([prompt], SamplingParams(ignore_eos=True))[0].token_ids == want, "the engine goes on"
