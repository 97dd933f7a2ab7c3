"""YAML configuration front-end.

Behaviour kept from the reference (savanna/arguments/arguments.py:94-1391):
  * several YAML files are merged; a key that appears in two files is an error (:171-174);
  * `-` and `_` are interchangeable in key names (:176-179);
  * unknown keys are rejected, values are type-checked (incl. Literal / Union) and range-checked;
  * derived values: world / data-parallel size, the batch triple, `save_iters`, precision, ZeRO
    settings, optimizer type and lr, `operator_config` expansion and context-parallel legality;
  * the resolved configuration is handed to the workers as base64 JSON (:500-581, :426-455);
  * the raw YAML text is kept in `config_files` so a checkpoint can store it verbatim.

The implementation is table driven (see schema.py): a `GlobalConfig` is a plain attribute bag whose
legal attribute set is the schema.
"""
from __future__ import annotations

import argparse
import base64
import copy
import json
import os
import typing
from typing import Any, Dict, Iterable, List, Optional

import yaml

from . import schema
from .schema import FIELDS, OPERATOR_CHOICES, OPT_DEFAULT, OPT_PARAMS_DEFAULTS, ZERO_DEFAULTS


class ConfigError(ValueError):
    pass


# ----------------------------------------------------------------------------- helpers


def expand_operator_types(operator_config, num_layers: int) -> List[str]:
    """Expand the compact `[[["a","b"], n], ...]` form (or `[[[...], "all"]]`) to one name per layer.

    Reference: savanna/utils.py:673-699.  A flat list of names is returned unchanged.
    """
    if all(isinstance(item, str) for item in operator_config):
        return list(operator_config)
    out: List[str] = []
    for item in operator_config:
        names, reps = item
        if reps == "all":
            if len(operator_config) != 1:
                raise ConfigError('"all" must be the only entry of operator_config')
            reps_n = num_layers // len(names)
            out = list(names) * reps_n + list(names)[: num_layers - reps_n * len(names)]
            return out
        for _ in range(int(reps)):
            out.extend(names)
    return out


def batch_triple(dp: int, train_batch=None, micro_batch=None, grad_acc=None):
    """Fill in whichever of (global batch, micro batch, accumulation steps) is missing."""
    if train_batch is not None and micro_batch is not None and grad_acc is not None:
        pass
    elif train_batch is not None and micro_batch is not None:
        grad_acc = train_batch // micro_batch // dp
    elif train_batch is not None and grad_acc is not None:
        micro_batch = train_batch // dp // grad_acc
    elif micro_batch is not None and grad_acc is not None:
        train_batch = micro_batch * grad_acc * dp
    elif train_batch is not None:
        grad_acc = 1
        micro_batch = train_batch // dp
    elif micro_batch is not None:
        grad_acc = 1
        train_batch = micro_batch * dp
    else:
        raise ConfigError("train_batch_size or train_micro_batch_size_per_gpu must be given")
    train_batch, micro_batch, grad_acc = int(train_batch), int(micro_batch), int(grad_acc)
    if min(train_batch, micro_batch, grad_acc) <= 0:
        raise ConfigError(f"batch parameters must be positive: {train_batch}, {micro_batch}, {grad_acc}")
    if train_batch != micro_batch * grad_acc * dp:
        raise ConfigError(
            f"train_batch_size {train_batch} != micro {micro_batch} * accumulation {grad_acc} * data-parallel {dp}"
        )
    return train_batch, micro_batch, grad_acc


def _type_ok(value, typ) -> bool:
    if value is None:
        return True
    origin = typing.get_origin(typ)
    if origin is typing.Literal:
        return value in typing.get_args(typ)
    if origin is typing.Union:
        return any(_type_ok(value, t) for t in typing.get_args(typ))
    if origin in (list, typing.List):
        return isinstance(value, (list, tuple))
    if typ is float:
        return isinstance(value, (int, float)) and not isinstance(value, bool)
    if typ is int:
        return isinstance(value, int) and not isinstance(value, bool)
    if typ is bool:
        return isinstance(value, bool)
    if typ is list:
        return isinstance(value, (list, tuple))
    if typ is dict:
        return isinstance(value, dict)
    if typ is str:
        return isinstance(value, str)
    return True


_GIT_DESCRIBE = []


def _git_describe() -> Optional[str]:
    """`git describe --always` of the checkout that holds this package (None outside a repository); asked once."""
    if not _GIT_DESCRIBE:
        import subprocess
        try:
            out = subprocess.run(["git", "describe", "--always"], cwd=os.path.dirname(os.path.abspath(__file__)),
                                 capture_output=True, text=True, timeout=10)
            _GIT_DESCRIBE.append(out.stdout.strip() or None if out.returncode == 0 else None)
        except Exception:
            _GIT_DESCRIBE.append(None)
    return _GIT_DESCRIBE[0]


def _detect_num_gpus() -> int:
    if "WORLD_SIZE" in os.environ:
        return int(os.environ["WORLD_SIZE"])
    try:
        import torch

        n = torch.cuda.device_count()
        return n if n > 0 else 1
    except Exception:
        return 1


# ----------------------------------------------------------------------------- GlobalConfig


class GlobalConfig:
    """Resolved configuration.  Attribute names are the schema keys plus a few derived ones."""

    _DERIVED = ("causal", "tokenizer", "tensorboard_writer", "dp_world_size")

    def __init__(self, **kwargs):
        unknown = sorted(k for k in kwargs if k not in FIELDS)
        if unknown:
            raise ConfigError(f"unknown configuration keys: {unknown}")
        for name, f in FIELDS.items():
            object.__setattr__(self, name, copy.deepcopy(kwargs.get(name, f.default)))
        self._explicit = set(kwargs)
        self.causal = True
        self.tokenizer = None
        self.tensorboard_writer = None
        self.validate_types()          # user-supplied values first, so derivation never sees a wrong type
        self.calculate_derived()
        self.validate_types()
        self.validate_values()

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_ymls(cls, paths: Iterable[str], overwrite_values: Optional[Dict] = None) -> "GlobalConfig":
        merged: Dict[str, Any] = {}
        files: Dict[str, str] = {}
        for path in paths:
            with open(path) as fh:
                text = fh.read()
            doc = yaml.load(text, Loader=yaml.FullLoader) or {}
            if not isinstance(doc, dict):
                raise ConfigError(f"{path}: top level of a config file must be a mapping")
            for key, value in doc.items():
                norm = key.replace("-", "_")
                if norm in merged:
                    raise ConfigError(f"{path}: key {key!r} was already set by an earlier config file")
                merged[norm] = value
            base = os.path.basename(path)
            if base in files:
                raise ConfigError(f"two config files share the name {base!r}; names must be unique")
            files[base] = text
        merged["config_files"] = files
        if overwrite_values:
            merged.update({k.replace("-", "_"): v for k, v in overwrite_values.items()})
        return cls(**merged)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GlobalConfig":
        return cls(**{k.replace("-", "_"): v for k, v in d.items()})

    @classmethod
    def defaults(cls) -> Dict[str, Any]:
        return {k: copy.deepcopy(f.default) for k, f in FIELDS.items()}

    # ------------------------------------------------------------------ mutation
    def update_value(self, key: str, value: Any) -> None:
        if key not in FIELDS and key not in self._DERIVED:
            raise ConfigError(f"unknown configuration key {key!r}")
        object.__setattr__(self, key, value)

    def update_values(self, d: Dict[str, Any]) -> None:
        for k, v in d.items():
            self.update_value(k, v)

    def __setattr__(self, key, value):
        if key.startswith("_") or key in FIELDS or key in self._DERIVED:
            object.__setattr__(self, key, value)
        else:
            raise ConfigError(f"unknown configuration key {key!r}")

    # ------------------------------------------------------------------ derived values
    def calculate_derived(self) -> None:
        n_gpus = self.global_num_gpus
        if n_gpus is None:
            n_gpus = self.num_gpus if (self.num_gpus or 0) > 0 and self.hostfile is None else _detect_num_gpus()
            self.global_num_gpus = n_gpus
        pp = max(1, self.pipe_parallel_size or 0)
        mp = max(1, self.model_parallel_size or 1)
        cp = max(1, self.context_parallel_size or 1)
        self.model_parallel_size = mp
        self.context_parallel_size = cp
        if n_gpus % (pp * mp * cp) != 0:
            raise ConfigError(
                f"{n_gpus} GPUs cannot be split into pipe {pp} x model {mp} x context {cp} groups"
            )
        dp = n_gpus // (pp * mp * cp)
        self.dp_world_size = dp
        self.world_size = n_gpus
        tb, mb, ga = batch_triple(
            dp, self.train_batch_size, self.train_micro_batch_size_per_gpu,
            self.gradient_accumulation_steps if "gradient_accumulation_steps" in self._explicit
            or self.train_batch_size is None or self.train_micro_batch_size_per_gpu is None else None,
        )
        self.train_batch_size, self.train_micro_batch_size_per_gpu, self.gradient_accumulation_steps = tb, mb, ga
        self.batch_size = mb
        self.gas = ga
        self.clip_grad = self.gradient_clipping

        # checkpoint schedule
        if self.checkpoint_factor or self.extra_save_iters:
            iters = set(self.extra_save_iters or [])
            step = self.checkpoint_factor
            if step:
                limit = self.train_iters or 0
                while step < limit:
                    iters.add(step)
                    step = step * self.checkpoint_factor if self.checkpoint_scale == "log" else step + self.checkpoint_factor
                    if self.checkpoint_scale == "log" and self.checkpoint_factor <= 1:
                        break
            self.save_iters = sorted(iters)

        # precision
        if self.fp16 and self.fp16.get("enabled", False):
            if self.precision not in (None, "fp16"):
                raise ConfigError("fp16.enabled conflicts with precision")
            self.precision = "fp16"
        if self.bf16 and self.bf16.get("enabled", False) and self.precision is None:
            self.precision = "bfloat16"
        if self.precision == "fp16":
            d = dict(self.fp16 or {"type": "fp16"})
            d["enabled"] = True
            self.fp16 = d
        elif self.precision == "bfloat16":
            extra = dict(self.deepspeed_extra_args or {})
            extra["bf16"] = {"enabled": True}
            self.deepspeed_extra_args = extra
        elif self.precision is None:
            self.precision = "fp32"

        # ZeRO
        if self.zero_optimization is None:
            self.zero_optimization = copy.deepcopy(ZERO_DEFAULTS)
        z = self.zero_optimization
        if "stage" not in z:
            raise ConfigError("zero_optimization needs a 'stage'")
        if z["stage"] not in (0, 1, 2, 3):
            raise ConfigError(f"zero stage must be 0..3, got {z['stage']!r}")
        self.zero_stage = z["stage"]
        self.zero_overlap_comm = bool(z.get("overlap_comm", ZERO_DEFAULTS["overlap_comm"]))
        self.zero_reduce_scatter = z.get("reduce_scatter", ZERO_DEFAULTS["reduce_scatter"])
        self.zero_contiguous_gradients = z.get("contiguous_gradients", ZERO_DEFAULTS["contiguous_gradients"])
        self.zero_reduce_bucket_size = int(z.get("reduce_bucket_size", ZERO_DEFAULTS["reduce_bucket_size"]))
        self.zero_allgather_bucket_size = int(z.get("allgather_bucket_size", ZERO_DEFAULTS["allgather_bucket_size"]))

        # optimizer
        opt = self.optimizer or {"type": OPT_DEFAULT, "params": dict(OPT_PARAMS_DEFAULTS)}
        self.optimizer_type = str(opt.get("type", OPT_DEFAULT)).lower()
        self.lr = opt.get("params", {}).get("lr", OPT_PARAMS_DEFAULTS["lr"])
        self.dynamic_loss_scale = self.loss_scale is None
        if self.git_hash is None:
            self.git_hash = _git_describe()         # recorded in the saved configuration next to every checkpoint

        self.is_pipe_parallel = (self.pipe_parallel_size or 0) > 1
        self.is_context_parallel = cp > 1

        # operators
        if self.num_layers is not None:
            oc = self.operator_config if self.operator_config is not None else [[["global"], self.num_layers]]
            oc = expand_operator_types(oc, self.num_layers)
            oc = ["hyena" if o == "hyena_li" else o for o in oc]
            if len(oc) != self.num_layers:
                raise ConfigError(f"operator_config expands to {len(oc)} layers, num_layers is {self.num_layers}")
            for o in oc:
                if o not in OPERATOR_CHOICES:
                    raise ConfigError(f"operator {o!r} is not known")
            if self.is_context_parallel:
                hyena_ops = {"hyena", "hyena_mr", "hyena_se"}
                if self.use_cp_flash_te:
                    legal = hyena_ops | {"flash_te"}
                elif self.use_cp_ring:
                    legal = hyena_ops | {"ring"}
                elif self.use_cp_hyena:
                    legal = hyena_ops | {"ring", "flash_te"}
                else:
                    raise ConfigError(
                        "context parallelism needs use_cp_hyena, use_cp_ring or use_cp_flash_te"
                    )
                bad = sorted(set(oc) - legal)
                if bad:
                    raise ConfigError(f"operators {bad} have no context-parallel algorithm")
                if self.is_pipe_parallel:
                    raise ConfigError("pipeline and context parallelism cannot be combined")
            self.operator_config = oc

        self.causal = self.pretraining_strategy == "AR"
        if self.sparsity_config is None:
            self.sparsity_config = {}
        for split in ("train", "valid", "test"):
            paths = getattr(self, f"{split}_data_paths")
            if paths and getattr(self, f"{split}_data_weights") is None:
                setattr(self, f"{split}_data_weights", [1.0] * len(paths))
        if self.text_gen_type is None:
            self.text_gen_type = "input-file" if self.sample_input_file else "unconditional"
        if self.rmsnorm_form is None:
            self.rmsnorm_form = "te" if self.use_fp8_norm else "classic"
        if self.max_position_embeddings is None and self.seq_length is not None:
            self.max_position_embeddings = self.seq_length
        if self.lr_decay_iters is None and self.train_iters is not None:
            self.lr_decay_iters = self.train_iters

    # ------------------------------------------------------------------ validation
    def validate_types(self) -> None:
        for name, f in FIELDS.items():
            value = getattr(self, name)
            if not _type_ok(value, f.type):
                raise ConfigError(f"config key {name!r}: value {value!r} is not of type {f.type}")

    def validate_values(self) -> None:
        if self.num_layers is None:
            return  # a partial configuration (e.g. data only); nothing model-related to check
        req = ("hidden_size", "num_attention_heads", "seq_length", "max_position_embeddings")
        missing = [k for k in req if getattr(self, k) is None]
        if missing:
            raise ConfigError(f"missing required keys: {missing}")
        if self.hidden_size % self.num_attention_heads:
            raise ConfigError("hidden_size must be divisible by num_attention_heads")
        if self.num_attention_heads % self.model_parallel_size:
            raise ConfigError("num_attention_heads must be divisible by model_parallel_size")
        if self.seq_length > self.max_position_embeddings and self.pos_emb == "learned":
            raise ConfigError("seq_length exceeds max_position_embeddings")
        if self.sequence_parallel and self.model_parallel_size <= 1:
            # harmless: sequence parallelism over a tensor-parallel group of one is the identity
            pass
        if self.context_parallel_size > 1 and self.seq_length % (2 * self.context_parallel_size):
            raise ConfigError("seq_length must be divisible by 2*context_parallel_size (zigzag sharding)")
        if self.lr_decay_iters is None and self.train_iters is None and self.do_train:
            raise ConfigError("train_iters or lr_decay_iters required")
        if not 0.0 <= (self.warmup or 0.0) <= 1.0:
            raise ConfigError("warmup is a fraction of the decay iterations and must lie in [0,1]")
        if self.optimizer_type not in typing.get_args(FIELDS["optimizer_type"].type):
            raise ConfigError(f"optimizer type {self.optimizer_type!r} is not supported")
        hyena_layers = [o for o in self.operator_config if o.startswith("hyena")]
        if hyena_layers:
            if self.short_conv_L is None:
                raise ConfigError("hyena layers need short_conv_L (featurizer filter length)")
            for key in ("num_groups_hyena", "num_groups_hyena_medium", "num_groups_hyena_short"):
                g = getattr(self, key)
                if g is not None and (self.hidden_size % g or g % self.model_parallel_size):
                    raise ConfigError(f"{key}={g} must divide hidden_size and be divisible by model_parallel_size")

    # ------------------------------------------------------------------ views
    def to_dict(self, only_non_default: bool = False) -> Dict[str, Any]:
        out = {}
        for name, f in FIELDS.items():
            v = getattr(self, name)
            if only_non_default and v == f.default:
                continue
            out[name] = v
        return out

    @property
    def engine_config(self) -> Dict[str, Any]:
        """The DeepSpeed-format dictionary (stored as `ds_config` in checkpoints)."""
        out = {}
        for k in schema.ENGINE_KEYS:
            v = getattr(self, k)
            if v is None or k in ("deepspeed", "deepspeed_extra_args"):
                continue
            out[k] = v
        if self.deepspeed_extra_args:
            out.update(self.deepspeed_extra_args)
        return out

    deepspeed_config = engine_config

    @property
    def params_dtype(self):
        import torch

        return {"fp16": torch.float16, "bfloat16": torch.bfloat16, "fp8": torch.bfloat16}.get(self.precision, torch.float32)

    @property
    def ffn_size(self) -> int:
        """Inner size of the gated MLP: explicit `ffn_hidden_size`, else the reference formula
        (savanna/model/operators/local/base.py:115-125)."""
        if self.ffn_hidden_size is not None:
            return int(self.ffn_hidden_size)
        m = self.make_gated_mlp_multiple_of
        ff = int(2 * self.hidden_size * 4 / 3)
        return m * ((ff + m - 1) // m)

    def print(self) -> None:
        width = max(len(k) for k in FIELDS)
        for name in sorted(FIELDS):
            v = getattr(self, name)
            if name == "config_files":
                v = list((v or {}).keys())
            mark = "" if v == FIELDS[name].default else "  (set)"
            print(f"  {name.ljust(width, '.')} {v}{mark}", flush=True)

    def save_yml(self, path: str) -> None:
        with open(path, "w") as fh:
            yaml.safe_dump(json.loads(json.dumps(self.to_dict(only_non_default=True), default=str)), fh)

    # ------------------------------------------------------------------ CLI (launch side)
    @classmethod
    def consume_deepy_args(cls, argv: Optional[List[str]] = None) -> "GlobalConfig":
        """Parse `launch.py <user_script> [-d conf_dir] a.yml b.yml ...` (arguments.py:235-424)."""
        p = argparse.ArgumentParser(description="savanna_b200 launcher", allow_abbrev=False)
        p.add_argument("user_script", type=str)
        p.add_argument("--conf_dir", "-d", type=str, default=None)
        p.add_argument("conf_file", type=str, nargs="+")
        p.add_argument("--wandb_group", type=str, default=None)
        p.add_argument("--wandb_team", type=str, default=None)
        p.add_argument("--wandb_project", type=str, default=None)
        p.add_argument("--wandb_run_name", type=str, default=None)
        p.add_argument("--eval_tasks", type=str, nargs="+", default=None)
        p.add_argument("--iteration", type=int, default=None)
        p.add_argument("--eval_results_prefix", type=str, default=None)
        p.add_argument("--hostfile", type=str, default=None)
        p.add_argument("--num_gpus", type=int, default=None)
        p.add_argument("--master_port", type=int, default=None)
        p.add_argument("--sample_input_file", "-i", type=str, default=None)
        p.add_argument("--sample_output_file", "-o", type=str, default=None)
        p.add_argument("--train-args-output", dest="train_args_output", type=str, default=None)
        p.add_argument("--overrides", type=str, default=None,
                       help="YAML file of KEY: VALUE pairs that replace values of the configuration files (the files "
                            "themselves may not set a key twice)")
        a = p.parse_args(argv)
        paths = []
        for f in a.conf_file:
            if not f.endswith((".yml", ".yaml", ".json")):
                f += ".yml"
            paths.append(os.path.join(a.conf_dir, f) if a.conf_dir else f)
        over = {
            k: getattr(a, k)
            for k in ("wandb_group", "wandb_team", "wandb_project", "wandb_run_name", "eval_tasks", "iteration",
                      "eval_results_prefix", "hostfile", "num_gpus", "master_port", "sample_input_file",
                      "sample_output_file")
            if getattr(a, k) is not None
        }
        over["user_script"] = a.user_script
        if a.overrides:
            path = os.path.join(a.conf_dir, a.overrides) if a.conf_dir and not os.path.isabs(a.overrides) \
                and not os.path.exists(a.overrides) else a.overrides
            with open(path) as fh:
                extra = yaml.load(fh, Loader=yaml.FullLoader) or {}
            if not isinstance(extra, dict):
                raise ConfigError(f"{path}: an overrides file holds a mapping of keys to values")
            over = {**extra, **over}
        cfg = cls.from_ymls(paths, overwrite_values=over)
        cfg._train_args_output = a.train_args_output
        return cfg

    def encoded(self) -> str:
        payload = self.to_dict(only_non_default=True)
        for k in ("tokenizer", "tensorboard_writer"):
            payload.pop(k, None)
        payload["global_num_gpus"] = self.global_num_gpus
        return base64.urlsafe_b64encode(json.dumps(payload, default=str).encode()).decode()

    def get_deepspeed_main_args(self) -> List[str]:
        """argv handed to the per-node launcher: runner flags, user script, encoded configs."""
        args: List[str] = []
        for k in schema.RUNNER_KEYS:
            v = getattr(self, k)
            if v is None or v is False or v == FIELDS[k].default:
                continue
            args += [f"--{k}"] if v is True else [f"--{k}", str(v)]
        args.append(self.user_script)
        ds = base64.urlsafe_b64encode(json.dumps(self.engine_config, default=str).encode()).decode()
        args += ["--deepspeed_config", ds, "--megatron_config", self.encoded()]
        return args

    get_launch_args = get_deepspeed_main_args

    # ------------------------------------------------------------------ CLI (worker side)
    @classmethod
    def consume_global_config(cls, argv: Optional[List[str]] = None, overwrite_values: Optional[Dict] = None):
        """Worker entry: decode `--megatron_config <b64>` (arguments.py:426-455)."""
        p = argparse.ArgumentParser(allow_abbrev=False)
        p.add_argument("--megatron_config", type=str, required=True)
        p.add_argument("--deepspeed_config", type=str, default=None)
        p.add_argument("--local_rank", type=int, default=None)
        a, _ = p.parse_known_args(argv)
        raw = a.megatron_config
        if os.path.isfile(raw):
            raw = open(raw).read().strip()
        d = json.loads(base64.urlsafe_b64decode(raw).decode())
        if overwrite_values:
            d.update(overwrite_values)
        cfg = cls.from_dict(d)
        cfg.configure_distributed_args()
        return cfg

    def configure_distributed_args(self) -> None:
        env = os.environ
        if "SLURM_PROCID" in env and "RANK" not in env:
            env["RANK"] = env["SLURM_PROCID"]
            env["LOCAL_RANK"] = env.get("SLURM_LOCALID", "0")
            env["WORLD_SIZE"] = env.get("SLURM_NTASKS", "1")
        self.local_rank = int(env.get("LOCAL_RANK", "0"))
        self.rank = int(env.get("RANK", "0"))
        self.world_size = int(env.get("WORLD_SIZE", "1"))

    def build_tokenizer(self) -> None:
        from ..data.tokenizer import build_tokenizer

        self.tokenizer = build_tokenizer(self)

    def initialize_tensorboard_writer(self) -> None:
        if self.tensorboard_dir and (self.rank or 0) == 0:
            try:
                from torch.utils.tensorboard import SummaryWriter

                self.tensorboard_writer = SummaryWriter(log_dir=self.tensorboard_dir)
            except Exception as exc:  # tensorboard is optional
                print(f"tensorboard unavailable ({exc}); continuing without it", flush=True)
