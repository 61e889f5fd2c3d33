"""The toy model of tests/test_toy_mixer_gpu.py (a mixer with a state of its own per request, a
block that runs twice, an architecture registered from the test) on the CPU, with the stand-in
kernels: registration, building, weight naming, state slots and stepping in portions need no GPU to
be checked, only the kernels do."""
import standin_ops
import test_toy_mixer_gpu


def test_toy_state_mixer_registers_builds_and_steps_on_the_host(tmp_path):
    test_toy_mixer_gpu.run_toy_model(tmp_path, device="cpu", ops=standin_ops)
