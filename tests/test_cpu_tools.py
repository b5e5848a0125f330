"""Launch, finetune and serving tools on CPU."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_slurm_launcher_writes_a_consistent_job(tmp_path):
    import launch_slurm as L

    job = L.parse_and_execute(["--config", "launch_configs/nebel_dp_8xb200.yaml", "--nodes", "4", "--budget_hours", "30",
                               "--timeslot", "720", "--dryrun", "--output_dir", str(tmp_path), "--run_name", "t",
                               "--overwrite_env", "NCCL_DEBUG=INFO FOO=1"])
    text = open(os.path.join(job.log_dir, "t.sbatch")).read()
    assert "#SBATCH --nodes=4" in text and "#SBATCH --gpus-per-node=8" in text and "#SBATCH --time=0-12:00:00" in text
    assert "--nnodes=4 --nproc-per-node=8" in text and "train.py --config=launch_configs/nebel_dp_8xb200.yaml" in text
    assert "export NCCL_DEBUG=INFO" in text and "export FOO=1" in text
    assert L.repetitions_needed(1800, 720) == 3
    cmds = L.submit(job, 3, use_chain=True, dryrun=True)
    assert len(cmds) == 3 and "afterany" in cmds[1]
    assert "salloc --nodes=4" in L.interactive(job)


def test_finetuning_example_learns():
    import finetuning_simple_example as F

    cfg = F.CLISettings(model_name="tiny", dataset_location="synthetic", max_steps=6, batch_size=4, micro_batch_size=2,
                        max_samples=32, max_seq_length=256, optim_config=dict(lr=3e-3, weight_decay=0.0))
    res = F.train(cfg)
    assert res["steps"] == 6 and res["losses"][-1] < 0.7 * res["losses"][0]
    assert abs(F.wsd_lr(0, 100, 1.0, 0.1, 0.1, 0.001) - 0.1) < 1e-9
    assert F.wsd_lr(50, 100, 1.0, 0.1, 0.1, 0.001) == 1.0 and F.wsd_lr(99, 100, 1.0, 0.1, 0.1, 0.001) < 0.2
    ids, mask = F.tokenize([("a?", "b")], F.ByteTokenizer(), cfg)
    assert mask.sum() == 3 and ids[0, 0] == F.ByteTokenizer.bos  # answer byte + end-of-turn + eos are supervised


def _tiny_hf():
    from recurrent_pretraining_b200.models.hf import RavenForCausalLM
    from recurrent_pretraining_b200.models.hf_config import RavenConfig

    torch.manual_seed(0)
    return RavenForCausalLM(RavenConfig(n_embd=64, n_heads=4, n_layers=4, block_size=64, vocab_size=128,
                                        intermediate_size=96, n_layers_in_recurrent_block=2, n_layers_in_prelude=1,
                                        n_layers_in_coda=1, mean_recurrence=3)).eval()


def test_server_batches_and_matches_direct_generation():
    from recurrent_pretraining_b200.engine import server as S

    model = _tiny_hf()
    sched = S.BatchScheduler(S.ModelBackend(model, max_batch=4), window_ms=50.0, stop_ids=())
    try:
        prompts = [[1, 2, 3, 4], [9, 8, 7, 6], [5, 5, 5]]
        reqs = [sched.submit(p, S.DecodeOptions(max_tokens=5, num_steps=3, init_scale=0.0)) for p in prompts]
        for r in reqs:
            assert r.done.wait(120) and r.error is None, r.error
        # the two 4-token prompts share a batch; the 3-token prompt runs alone
        assert sched.stats["requests"] == 3 and sched.stats["batches"] == 2
        for p, r in zip(prompts, reqs):
            want = model.generate(torch.tensor([p]), max_new_tokens=5, num_steps=3, init_scale=0.0)
            want = (want["sequences"] if isinstance(want, dict) else want)[0, len(p):].tolist()
            assert r.tokens == want
        out = S.handle_completion(sched, {"prompt": [1, 2, 3, 4], "max_tokens": 3, "num_steps": 2})
        assert out["usage"] == {"prompt_tokens": 4, "completion_tokens": 3, "total_tokens": 7}
        assert out["choices"][0]["finish_reason"] == "length"
        app = S.create_app(sched)
        assert {r.path for r in app.routes} >= {"/health", "/v1/models", "/v1/completions"}
        try:
            S.handle_completion(sched, {"prompt": "text without tokenizer"})
            raise AssertionError("expected a ValueError")
        except ValueError:
            pass
    finally:
        sched.close()


def test_example_scripts_run():
    import examples.inference_demo as demo
    import examples.speculative_decoding_demo as spec

    demo.main(["--max_new_tokens", "3"])
    spec.main()
    import examples.trajectory_analysis as traj

    rows = traj.main(["--steps", "6", "--tokens", "3"])
    assert len(rows) == 3 and all(len(r["xy"]) == 7 for r in rows)
