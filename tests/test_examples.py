"""The example programs double as acceptance tests."""
import importlib.util
import os


def _load(name):
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples",
                        name + ".py")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_ping_pong_and_dining_philosophers():
    out = _load("ping_pong").run(in_process=False)
    assert out["ping_hits"] == [4, 4]           # 6 bounces + the serve end on the ping side
    assert out["meals"] == [3] * 5
    assert 1 <= out["max_eating_at_once"] <= 2  # never two neighbours at once


def test_grpo_weight_refresh_learns():
    out = _load("grpo_weight_refresh").run(iters=40)
    assert out["versions"] == 40
    assert out["reward_last"] > out["reward_first"] + 0.1, out


def test_distributed_tensor_ddp():
    out = _load("distributed_tensors_ddp").run()
    assert out["replicas_in_sync"]
    assert out["loss_last"] < out["loss_first"]


def test_llama_ddp_over_distributed_tensors_compiled_step():
    """The whole training step (forward, controller-side autograd, bucketed gradient
    all-reduce, foreach AdamW with the step count on the workers) as one recording."""
    out = _load("llama_ddp_distributed_tensors").run(
        model="tiny", procs=2, cuda=False, seq=32, micro_batch=2, steps=3, warmup=2)
    assert out["replicas_in_sync"] and out["compiled"]
    assert out["loss_last"] < out["loss_first"]


def test_lazy_top_level_api():
    import monarch_b200 as m
    assert m.DeviceMesh is m.tensor_engine.DeviceMesh and callable(m.remote)
    assert "fetch_shard" in dir(m) and m.timer.CudaTimer


def test_sieve_of_dynamically_spawned_actors():
    out = _load("sieve").run(15)
    assert out["primes"] == [2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37, 41, 43, 47]


def test_rdma_parameter_server_converges():
    out = _load("rdma_parameter_server").run(n_workers=2, steps=60)
    assert out["loss_last"] < 1e-3 * out["loss_first"], out
    assert out["weight_error"] < 0.05


def test_spmd_ddp_inside_actors():
    out = _load("spmd_ddp").run(world_size=2, steps=30)
    assert out["replicas_in_sync"], out
    assert out["loss_last"] < 0.5 * out["loss_first"], out


def test_getting_started_tour():
    out = _load("getting_started").run()
    assert out["values"] == [2, 2, 1, 1] and out["registered"] == 2
    assert out["supervision_event"] == "actor_failed" and out["caller_error"]


def test_fsdp_training_driven_over_an_actor_mesh():
    out = _load("fsdp_on_mesh").run(model="tiny", gpus=2, seq=32, steps=4, use_cuda=False)
    assert len(out["losses_first"]) == 2
    first = sum(out["losses_first"]) / 2
    last = sum(out["losses_last"]) / 2
    assert last < first, out          # the sharded optimizer step learns


def test_distributed_tensors_tour():
    out = _load("distributed_tensors").run()
    assert out["error_caught"] and out["pipeline_out"] == 16.0
    assert out["coords"] == [[0, 1], [10, 11]] and out["compiled"] == (189.0, 189.0)
