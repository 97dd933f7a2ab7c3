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
