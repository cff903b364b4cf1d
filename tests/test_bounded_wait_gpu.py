"""A wait inside a kernel that runs out (GPU): the kernel returns, the status word says so, the step
function turns it into an exception, and the context goes on working.  The wait is the kernels' own
bounded mbarrier wait (csrc/mbarrier.cuh) with a limit of a few hundred polls, on a barrier on which
nothing arrives; it ends by itself after microseconds."""
import pytest
import torch

import plain_model
import tiny_configs

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_sets_the_status_bit_and_returns():
    from easy_gpt.cpp_b200 import kernels

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for threads, limit in ((1, 10), (32, 300), (192, 1000)):
        assert kernels.wait_probe(limit, threads, status) == threads       # every thread left its wait
        assert status.item() == 8
        assert "bounded wait" in kernels.describe_status(int(status.item()))
        status.zero_()
    with pytest.raises(kernels.KernelError):
        kernels.wait_probe(0, 32, status)                                  # refused: a limit of at least one poll


def test_the_step_function_reports_it_and_goes_on(tmp_path):
    from easy_gpt.cpp_b200 import kernels
    from easy_gpt.cpp_b200.engine import Model, StepEntry, StepError, StepRunner

    folder = tiny_configs.write_tiny("C", tmp_path / "m")
    model = Model.from_dir(folder, device="cuda:0", dtype=torch.bfloat16)
    runner = StepRunner(model, page_size=16, num_pages=16, max_slots=2)
    tokens = tiny_configs.random_tokens(203, 90, 1)
    first = runner.run([StepEntry("a", tokens[:50], [49])])
    kernels.wait_probe(200, 64, runner.status)                             # a kernel of the step gave up its wait
    with pytest.raises(StepError, match="bounded wait inside a kernel gave up"):
        runner.run([StepEntry("a", tokens[50:], [39])])
    runner.end("a")
    # the status word was cleared and the context still works: the same request again, whole
    again = runner.run([StepEntry("b", tokens[:50], [49])])
    assert torch.equal(first, again)
    cfg, w = plain_model.read_model_dir(folder, round_to_bf16=True)
    ref = plain_model.forward_logits(cfg, w, tokens[:50])[49]
    assert float((again[0].cpu() - ref).abs().max()) <= 1.5e-2 * float(ref.abs().max())
