"""The toy models of tests/test_toy_parts_gpu.py on the CPU, with the stand-in kernels: a feed-forward
that routes tokens to experts and a learned position encoding, a windowed layer beside a full one
(two cache groups, pages given back as the window passes), a layer that reads another layer's
cache.  Registration, building, weight naming, cache groups and the run order need no GPU to be
checked, only the kernels do (the GPU tests run the same models on them)."""
import standin_ops
import test_toy_parts_gpu as toys

HOST = dict(device="cpu", ops=standin_ops)


def test_routed_feed_forward_and_learned_positions_on_the_host(tmp_path):
    toys.run_routed_model(tmp_path, **HOST)


def test_windowed_layer_beside_a_full_one_on_the_host(tmp_path):
    toys.run_windowed_model(tmp_path, "float32", graphs=False, **HOST)


def test_layer_reading_another_layers_cache_on_the_host(tmp_path):
    toys.run_shared_cache_model(tmp_path, "float32", graphs=False, **HOST)
