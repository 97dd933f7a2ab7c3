"""SLURM script generation, configuration overrides, environment checks and the tuner's variant grid / job array."""
import os
import subprocess
import sys

import pytest
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_slurm_script_with_overrides_and_presets(tmp_path):
    from launcher import slurm
    conf = tmp_path / "conf"
    conf.mkdir()
    (conf / "model.yml").write_text("{}")
    out = tmp_path / "job.sbatch"
    cwd = os.getcwd()
    os.chdir(ROOT)
    try:
        slurm.main(["model.yml", "-d", str(conf), "--job-name", "evo", "--nodes", "2", "--gpus-per-node", "8", "--max-restarts", "3",
                    "--override", "train-iters=50", "--override", "zero_optimization={stage: 1, overlap_comm: true}",
                    "--checkpoint-dir", "/scratch/run1", "--straggler-interval", "20", "--watchdog-timeout", "600", "--nsys",
                    "--singleton", "--output", str(out)])
    finally:
        os.chdir(cwd)
    text = out.read_text()
    assert "#SBATCH --nodes=2" in text and "#SBATCH --dependency=singleton" in text and "--max-restarts=3" in text
    assert "nsys profile" in text and "--capture-range=cudaProfilerApi" in text
    assert "--overrides overrides-evo.yml" in text and "--train-args-output" in text
    over = yaml.safe_load((conf / "overrides-evo.yml").read_text())
    assert over["save"] == over["load"] == "/scratch/run1" and over["train-iters"] == 50
    assert over["zero_optimization"] == {"stage": 1, "overlap_comm": True}
    assert over["heimdall_log_straggler"] is True and over["heimdall_log_interval"] == 20
    assert over["watchdog_step_timeout"] == 600.0 and "heartbeat-evo" in over["watchdog_heartbeat_dir"]
    # launch.py applies the file on top of the configuration files
    from savanna_b200.config import GlobalConfig
    cfg = GlobalConfig.consume_deepy_args(["train.py", os.path.join(ROOT, "configs", "baseline", "tiny_sh2_cpu.yml"), "--num_gpus", "1",
                                           "--overrides", str(conf / "overrides-evo.yml")])
    assert cfg.train_iters == 50 and cfg.zero_overlap_comm and cfg.save == "/scratch/run1"


def test_slurm_env_check(tmp_path):
    from launcher.config_parser import check_slurm_env, world_info
    hf = tmp_path / "hosts"
    hf.write_text("node-a slots=8\nnode-b slots=8\n")
    env = {"SLURM_JOB_NUM_NODES": "2", "MASTER_NODE": "node-a", "MASTER_PORT": "29500", "SLURM_GPUS_ON_NODE": "8"}
    assert check_slurm_env(str(hf), env) == ("node-a", 2, 8)
    with pytest.raises(RuntimeError, match="3 nodes"):
        check_slurm_env(str(hf), dict(env, SLURM_JOB_NUM_NODES="3"))
    with pytest.raises(RuntimeError, match="not the first host"):
        check_slurm_env(str(hf), dict(env, MASTER_NODE="node-b"))
    import base64, json
    assert json.loads(base64.urlsafe_b64decode(world_info(["node-a", "node-b"], 2))) == {"node-a": [0, 1], "node-b": [0, 1]}


def test_tuner_grid_and_job_array(tmp_path):
    from tuner import tuner
    out = tmp_path / "runs"
    cwd = os.getcwd()
    os.chdir(ROOT)
    try:
        tuner.main(["generate", "--base", "configs/baseline/tiny_sh2_cpu.yml", "--gpus", "8", "--out", str(out), "--micro-batch", "1", "2",
                    "--tp", "1", "2", "--cp", "1", "4", "--checkpoint-num-layers", "0", "2", "--array", "--array-parallel", "4", "--nsys"])
    finally:
        os.chdir(cwd)
    names = (out / "variants.txt").read_text().split()
    assert len(names) == 16 and "mb2_tp2_cp4_ac2_z1" in names
    text = (out / "array.sbatch").read_text()
    assert "#SBATCH --array=0-15%4" in text and "SLURM_ARRAY_TASK_ID" in text and '"$TAG.yml"' in text and "nsys profile" in text
    cfg = yaml.safe_load((out / "configs" / "mb2_tp2_cp4_ac2_z1.yml").read_text())
    assert cfg["model_parallel_size"] == 2 and cfg["context_parallel_size"] == 4 and cfg["sequence_parallel"] and cfg["use_cp_hyena"]
    assert subprocess.run(["bash", "-n", str(out / "array.sbatch")]).returncode == 0          # the script parses


def test_ops_scripts_config_diff_log_parse_checkpoint_summary_filter_lens(tmp_path):
    import torch
    from launcher.scripts import compare_configs, filter_lens, parse_logs, summarize_checkpoints
    # config diff, raw and resolved
    a, b = tmp_path / "a.yml", tmp_path / "b.yml"
    a.write_text("{\n  \"hidden-size\": 64,\n  \"optimizer\": {\"type\": \"Adam\", \"params\": {\"lr\": 0.001}}\n}\n")
    b.write_text("{\n  \"hidden_size\": 128,\n  \"optimizer\": {\"type\": \"Adam\", \"params\": {\"lr\": 0.002}},\n  \"seed\": 3\n}\n")
    diffs = compare_configs.compare([str(a)], [str(b)])
    assert any(d.startswith("hidden_size differs") for d in diffs)
    assert any("optimizer/params/lr differs" in d for d in diffs) and any(d == "seed only in second" for d in diffs)
    # log scraping
    log = tmp_path / "train.log"
    log.write_text(" iteration       10/    1000 | lm_loss: 2.345E+00 | tokens/s/gpu: 4.1E+04 | lr: 1.0E-04 |\n"
                   "SAVE_CHECKPOINT: iteration: 10, ckpt saving takes 12.5 seconds\n"
                   " iteration       20/    1000 | lm_loss: 2.1E+00 | tokens/s/gpu: 4.2E+04 |\n"
                   "time (ms) | model and optimizer: 1234.5 | train/valid/test data iterators: 56.7\n")
    lines = log.read_text().splitlines()
    it = parse_logs.parse_iterations(lines)
    assert [r["iteration"] for r in it] == [10, 20] and it[0]["lm_loss"] == 2.345 and it[1]["tokens/s/gpu"] == 4.2e4
    ck = parse_logs.parse_checkpoint_times(lines)
    assert ck == [{"iteration": 10, "checkpoint_time": 12.5}]
    assert parse_logs.describe(ck, "checkpoint_time")["mean"] == 12.5
    assert parse_logs.parse_startup(lines)[0]["model_and_optimizer"] == 1234.5
    parse_logs.write_csv(it, str(tmp_path / "it.csv"))
    assert (tmp_path / "it.csv").read_text().startswith("iteration,train_iters,lm_loss")
    # checkpoint summary
    save = tmp_path / "save"
    for step, files in ((10, ["mp_rank_00_model_states.pt", "bf16_zero_pp_rank_0_mp_rank_00_optim_states.pt"]), (20, [])):
        d = save / f"global_step{step}"
        d.mkdir(parents=True)
        for f in files:
            (d / f).write_bytes(b"x" * 100)
    (save / "latest").write_text("global_step10")
    (save / "global_step10" / ".uploaded").write_text("")
    res = summarize_checkpoints.summarize(str(save), expect_mp=1, expect_dp=1)
    assert res["latest"] == "global_step10" and res["steps"][10]["complete"] and res["steps"][10]["uploaded"]
    assert 20 not in res["steps"] or not res["steps"][20]["complete"]
    # filter lengths: an un-padded checkpoint is reported, fixed, and then passes
    ck_dir = tmp_path / "ext"
    (ck_dir / "zero" / "sequential.3.mixer.mixer.filter.h").mkdir(parents=True)
    h = torch.randn(4, 16)
    torch.save({"module": {"sequential.3.mixer.mixer.filter.h": h.clone(), "other.weight": torch.ones(2)},
                "param_shapes": [{"sequential.3.mixer.mixer.filter.h": h.shape}]}, ck_dir / "mp_rank_00_model_states.pt")
    torch.save({"fp32": h.clone().flatten(), "exp_avg": torch.zeros(64)}, ck_dir / "zero" / "sequential.3.mixer.mixer.filter.h" / "fp32.pt")
    probs = filter_lens.check(str(ck_dir), 4, 16, 64)
    assert len(probs) >= 2
    changed = filter_lens.fix(str(ck_dir), 4, 16, 64)
    assert changed == {"model_tensors": 1, "zero_tensors": 2}
    probs = filter_lens.check(str(ck_dir), 4, 16, 64)
    assert probs == ["zero/sequential.3.mixer.mixer.filter.h/fp32.pt:exp_avg: only zeros in the filter region [0:16)"]
    sd = torch.load(ck_dir / "mp_rank_00_model_states.pt", weights_only=False)
    assert torch.equal(sd["module"]["sequential.3.mixer.mixer.filter.h"][:, :16], h) and sd["param_shapes"][0][
        "sequential.3.mixer.mixer.filter.h"] == torch.Size([4, 64])


def test_launch_command_with_per_rank_logs(tmp_path, monkeypatch):
    """`enable_each_rank_log`: the worker command redirects every rank's output into its own file under rank_logs."""
    import importlib.util
    from savanna_b200.config import GlobalConfig
    spec = importlib.util.spec_from_file_location("launch_mod", os.path.join(ROOT, "launch.py"))
    launch = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(launch)
    tiny = os.path.join(ROOT, "configs", "baseline", "tiny_sh2_cpu.yml")
    cfg = GlobalConfig.consume_deepy_args(["train.py", tiny, "--num_gpus", "2"])
    cmd = launch.build_command(cfg)
    assert "--log-dir" not in cmd and cmd[cmd.index("train.py") - 1] != "3"
    cfg.enable_each_rank_log = True
    cfg.log_dir = str(tmp_path / "logs")
    cmd = launch.build_command(cfg)
    i = cmd.index("--log-dir")
    assert cmd[i + 1] == os.path.join(str(tmp_path / "logs"), "rank_logs") and os.path.isdir(cmd[i + 1])
    assert cmd[i + 2: i + 6] == ["--redirects", "3", "--tee", "3"] and cmd.index("train.py") > i
    assert "--nproc-per-node=2" in cmd
