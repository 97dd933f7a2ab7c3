import json
import os

import numpy as np
import pytest
import torch

from savanna_b200.config import GlobalConfig
from savanna_b200.data.synthetic import acgt_batch
from savanna_b200.train.trainer import Trainer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = os.path.join(ROOT, "configs", "baseline", "tiny_sh2_cpu.yml")


@pytest.fixture()
def tiny_ckpt(tmp_path):
    from savanna_b200.ckpt import save_checkpoint
    cfg = GlobalConfig.from_ymls([TINY], {"global_num_gpus": 1, "save": str(tmp_path / "ck"),
                                          "zero_optimization": {"stage": 1}})
    tr = Trainer(cfg, load=False)
    tr.train_step(iter([{"text": acgt_batch(2, cfg.seq_length, 0)}]))
    return tr, save_checkpoint(tr)


def test_tp_reshard_roundtrip(tiny_ckpt, tmp_path):
    from savanna_b200.tools.reshard_model_parallel import load_shards, reshard
    tr, d = tiny_ckpt
    reshard(d, str(tmp_path / "mp4"), 4)
    parts = load_shards(str(tmp_path / "mp4"))
    assert len(parts) == 4
    assert parts[0]["module"]["sequential.2.mixer.dense_projection.weight"].shape == (192, 256)
    assert parts[0]["module"]["sequential.2.mixer.dense.weight"].shape == (256, 64)
    assert parts[0]["module"]["sequential.2.input_layernorm.weight"].shape == (256,)
    reshard(str(tmp_path / "mp4"), str(tmp_path / "mp1"), 1)
    back = load_shards(str(tmp_path / "mp1"))[0]["module"]
    for k, v in tr.model.state_dict().items():
        assert torch.equal(back[k], v.cpu()), k


def test_interleave_roundtrip():
    from savanna_b200.tools.interleave_model_states import deinterleave_rows, interleave_rows
    w = torch.arange(12 * 2).view(12, 2)
    i = interleave_rows(w)
    assert i[0].tolist() == w[0].tolist() and i[1].tolist() == w[4].tolist() and i[2].tolist() == w[8].tolist()
    assert torch.equal(deinterleave_rows(i), w)


def test_extend_filter(tiny_ckpt):
    from savanna_b200.tools.extend_filter import extend_module
    tr, _ = tiny_ckpt
    mod = {k: v.cpu() for k, v in tr.model.state_dict().items()}
    out = extend_module(mod, 4096, taps=128)
    h = out["sequential.3.mixer.mixer.filter.h"]
    assert h.shape == (16, 4096) and torch.equal(h[:, :128], mod["sequential.3.mixer.mixer.filter.h"][:, :128])
    assert out["sequential.3.mixer.mixer.filter.decay"].shape == (16, 4096)
    assert out["sequential.4.mixer.mixer.filter.t"].shape == (1, 1, 4096)


def test_zero_to_fp32_and_dp_reshard(tiny_ckpt, tmp_path):
    from savanna_b200.tools.reshard_zero import reshard
    from savanna_b200.tools.zero_to_fp32 import consolidate
    tr, d = tiny_ckpt
    sd = consolidate(d)
    for k, v in tr.model.state_dict().items():
        assert torch.allclose(sd[k].float(), v.float().cpu(), atol=1e-6), k
    reshard(d, str(tmp_path / "dp4"), 4)
    sd4 = consolidate(str(tmp_path / "dp4"))
    for k in sd:
        assert torch.equal(sd[k], sd4[k]), k


def test_vortex_export(tiny_ckpt):
    from savanna_b200.tools.convert_checkpoint_to_vortex import convert
    tr, _ = tiny_ckpt
    out = convert({k: v.cpu() for k, v in tr.model.state_dict().items()})
    for k in ("blocks.0.filter.h", "blocks.1.filter.h", "blocks.2.filter.log_poles", "blocks.2.filter.residues",
              "blocks.3.inner_mha_cls.Wqkv.weight", "blocks.0.mlp.l1.weight", "embedding_layer.weight", "norm.scale"):
        assert k in out, k
    assert out["blocks.1.filter.h"].shape == (16, 1, 128)


def test_preprocess_and_load(tmp_path):
    from savanna_b200.data.indexed_dataset import MMapIndexedDataset
    from savanna_b200.tools.preprocess_data import main
    src = tmp_path / "d.jsonl"
    src.write_text("\n".join(json.dumps({"text": t}) for t in ("ACGT", "GGGTTTAAAC", "T")) + "\n")
    main(["--input", str(src), "--output-prefix", str(tmp_path / "out"), "--append-eod"])
    ds = MMapIndexedDataset(str(tmp_path / "out_text_document"))
    assert len(ds) == 3 and ds[0].tolist() == [65, 67, 71, 84, 0] and ds[2].tolist() == [84, 0]
    # uniform-length data: only documents of exactly --enforce-sample-length tokens are kept; the older index format
    src2 = tmp_path / "u.jsonl"
    src2.write_text("\n".join(json.dumps({"text": t}) for t in ("ACGTACG", "ACG", "TTTTGGG", "ACGTACGTAC")) + "\n")
    main(["--input", str(src2), "--output-prefix", str(tmp_path / "uni"), "--append-eod", "--enforce-sample-length", "8",
          "--dataset-impl", "lazy", "--num-docs", "4", "--log-interval", "1"])
    from savanna_b200.data import indexed_dataset as ids
    assert ids.infer_dataset_impl(str(tmp_path / "uni_text_document")) in ("lazy", "cached")
    uni = ids.make_dataset(str(tmp_path / "uni_text_document"), "lazy")
    assert len(uni) == 2 and all(len(uni[i]) == 8 for i in range(2))
    # ... and trains as fixed-length samples: every sample is one whole document
    from savanna_b200.data.sequence_dataset import SequenceDataset
    import numpy as np
    sd = SequenceDataset("train", str(tmp_path / "uni_text_document"), np.arange(2, dtype=np.int32), uni, 2, 8, 1,
                         enforce_sample_length=True)
    assert len(sd) >= 1 and sd[0]["text"].shape == (9,)


def test_generation_greedy_is_deterministic():
    from savanna_b200.inference import generate
    cfg = GlobalConfig.from_ymls([TINY], {"global_num_gpus": 1})
    tr = Trainer(cfg, load=False)
    a = generate(tr.model, cfg.tokenizer, ["ACGT", "GG"], maximum_tokens=5)
    b = generate(tr.model, cfg.tokenizer, ["ACGT", "GG"], maximum_tokens=5)
    assert [r["text"] for r in a] == [r["text"] for r in b] and all(r["length"] >= 5 for r in a)


def test_generation_from_file_splits_prompts_at_prompt_end(tmp_path):
    from savanna_b200.inference.generation import generate_samples_input_from_file
    cfg = GlobalConfig.from_ymls([TINY], {"global_num_gpus": 1, "prompt_end": "<|end|>", "maximum_tokens": 3})
    tr = Trainer(cfg, load=False)
    src = tmp_path / "prompts.txt"
    src.write_text("ACGT\nACGT<|end|>GGCC<|end|>\n")
    out = tmp_path / "out.jsonl"
    res = generate_samples_input_from_file(tr.model, cfg, str(src), str(out))
    assert [r["context"] for r in res] == ["ACGT\nACGT", "GGCC"]
    assert len(out.read_text().strip().splitlines()) == 2
    assert isinstance(cfg.git_hash, (str, type(None)))


def test_convert_checkpoint_to_torch(tiny_ckpt, tmp_path):
    from savanna_b200.tools.convert_checkpoint_to_torch import convert
    tr, d = tiny_ckpt
    plain = convert(d, str(tmp_path / "model.pt"))
    assert os.path.exists(tmp_path / "model.pt")
    for k, v in tr.model.state_dict().items():
        assert torch.equal(plain[k], v.cpu()), k
    named = convert(d, str(tmp_path / "standalone.pt"), strip_prefix=True)
    assert "embedding.word_embeddings.weight" in named and "blocks.0.mixer.dense_projection.weight" in named
    assert any(k.startswith("final_norm.") for k in named)
    assert len(named) == len(plain)
    fp32 = convert(d, str(tmp_path / "fp32.pt"), fp32=True)
    k = "sequential.2.mixer.dense_projection.weight"
    assert fp32[k].dtype == torch.float32 and torch.allclose(fp32[k], plain[k].float(), atol=1e-2)


def test_load_for_inference_roundtrip(tiny_ckpt):
    """A saved checkpoint rebuilds the model from its stored configs and reproduces the trainer's logits."""
    from savanna_b200.inference.load import load_for_inference
    from savanna_b200.parallel import state
    tr, d = tiny_ckpt
    tokens = acgt_batch(1, 64, 5)[:, :64]
    tr.model.eval()
    with torch.no_grad():
        want = tr.model(tokens, torch.arange(64))
    state.destroy_model_parallel()
    model, tok, cfg = load_for_inference(os.path.dirname(d), config_files=[TINY])
    with torch.no_grad():
        got = model(tokens, torch.arange(64))
    assert torch.allclose(got, want, atol=1e-5)
    assert tok is not None and cfg.hidden_size == 256


def _byte_dataset(path, ndocs, seed, low, high):
    import numpy as np
    from savanna_b200.data.indexed_dataset import MMapIndexedDatasetBuilder
    rng = np.random.default_rng(seed)
    b = MMapIndexedDatasetBuilder(path + ".bin", dtype=np.uint16)
    for _ in range(ndocs):
        b.add_item(rng.integers(low, high, size=int(rng.integers(100, 400))))
        b.end_document()
    b.finalize(path + ".idx")
    return path


def test_evaluate_per_dataset_tool(tmp_path):
    """Two validation files give two separately reported losses; the in-training hook logs them under their names."""
    import os
    from savanna_b200.parallel import state
    from savanna_b200.tools import evaluate_per_ds
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tiny = os.path.join(root, "configs", "baseline", "tiny_sh2_cpu.yml")
    d1, d2 = tmp_path / "genomes" / "valid", tmp_path / "plasmids" / "valid"
    d1.mkdir(parents=True); d2.mkdir(parents=True)
    p1 = _byte_dataset(str(d1 / "data_text_document"), 40, 0, 65, 69)
    p2 = _byte_dataset(str(d2 / "data_text_document"), 40, 1, 97, 123)
    out = tmp_path / "res.json"
    state.destroy_model_parallel()
    res = evaluate_per_ds.main([tiny, "--iters", "2", "--json", str(out), "--override", "global_num_gpus=1",
                                "--override", f"per_ds_valid_data_paths=[{p1}, {p2}]", "--override", "synthetic_data=null",
                                "--override", f"train_data_paths=[{p1}]", "--override", "train_data_weights=[1.0]"])
    assert list(res) == ["genomes", "plasmids"]
    assert all(r["lm_loss"] == r["lm_loss"] and r["lm_loss"] > 0 for r in res.values())
    import json
    assert set(json.load(open(out))) == {"genomes", "plasmids"}
    assert "genomes" in evaluate_per_ds.format_table(res)
    state.destroy_model_parallel()


def test_parquet_to_json(tmp_path):
    import json
    import pyarrow as pa
    import pyarrow.parquet as pq
    from savanna_b200.tools import parquet_to_json
    src, dst = str(tmp_path / "a.parquet"), str(tmp_path / "a.jsonl")
    pq.write_table(pa.table({"text": ["ACGT", "GGCC", "TTAA"], "id": [1, 2, 3]}), src)
    assert parquet_to_json.main([src, dst, "--columns", "text"]) == 3
    rows = [json.loads(l) for l in open(dst)]
    assert rows == [{"text": "ACGT"}, {"text": "GGCC"}, {"text": "TTAA"}]


def test_ds_to_universal(tiny_ckpt, tmp_path):
    """Per-parameter export: every parameter's fp32 master and Adam moments come back whole, with a step file."""
    import os
    from savanna_b200.tools.ds_to_universal import convert, load_universal_param
    tr, d = tiny_ckpt
    out = str(tmp_path / "universal")
    names = convert(d, out, write_latest=False)
    sd = {n: p.detach() for n, p in tr.model.named_parameters()}
    assert set(names) == {n for n, p in tr.model.named_parameters() if p.requires_grad}
    for n in names:
        w = load_universal_param(out, n)
        assert w.shape == sd[n].shape and w.dtype == torch.float32
        assert torch.allclose(w, sd[n].float().cpu(), atol=1e-2, rtol=1e-2), n
        m = load_universal_param(out, n, "exp_avg")
        assert m.shape == sd[n].shape
        assert os.path.isfile(os.path.join(out, "zero", n, "step.pt"))
    assert os.path.isfile(os.path.join(out, "zero", "optimizer_state.pt"))
    assert os.path.isfile(os.path.join(out, "mp_rank_00_model_states.pt"))


def test_cached_generation_matches_recompute():
    """Constant-time decoding from cached layer state (FIR tails, modal states, key/value cache) reproduces the logits
    and the greedy continuation of re-running the model on the growing context."""
    from savanna_b200.inference.cached import CachedDecoder, stream_tokens_cached
    from savanna_b200.inference.generation import generate, generate_samples_interactive, stream_tokens
    from savanna_b200.models import build_model
    cfg = GlobalConfig.from_ymls([TINY], {"global_num_gpus": 1, "hidden_dropout": 0.0})
    cfg.build_tokenizer()
    torch.manual_seed(0)
    model = build_model(cfg)
    with torch.no_grad():                                  # make the state-dependent terms matter
        for n, p in model.named_parameters():
            if n.endswith("filter.h"):
                p.mul_(3e4)
    prompt = [[65, 67, 71, 84, 65, 65, 67, 71, 84, 84, 71, 67] * 12, [84, 71, 67, 65, 84, 84, 71, 67, 65, 65, 67, 71] * 12]
    ref_stream = list(stream_tokens(model, prompt, maximum_tokens=10))
    cached = list(stream_tokens_cached(model, prompt, maximum_tokens=10))
    assert len(ref_stream) == len(cached) == 10
    for (t_ref, _, l_ref, _), (t_c, l_c, _) in zip(ref_stream, cached):
        assert torch.equal(t_ref, t_c)
        assert torch.allclose(l_ref, l_c, atol=2e-3, rtol=2e-3), (l_ref - l_c).abs().max()
    # decoder API: prefill then single steps
    dec = CachedDecoder(model)
    toks = torch.tensor(prompt)
    l0 = dec.prefill(toks)
    assert torch.allclose(l0, model(toks)[:, -1].float(), atol=1e-4)
    nxt = l0.argmax(-1)
    l1 = dec.step(nxt)
    assert torch.allclose(l1, model(torch.cat([toks, nxt[:, None]], 1))[:, -1].float(), atol=2e-3, rtol=2e-3)
    # string-level drivers
    a = generate(model, cfg.tokenizer, ["ACGTACGTAC", "TTGACCAGTA"], maximum_tokens=8, use_cache=True)
    b = generate(model, cfg.tokenizer, ["ACGTACGTAC", "TTGACCAGTA"], maximum_tokens=8, use_cache=False)
    assert [r["text"] for r in a] == [r["text"] for r in b]
    said, prompts = [], iter(["ACGTACGT", ""])
    generate_samples_interactive(model, cfg, input_fn=lambda _: next(prompts), print_fn=lambda *x, **k: said.append(x[0]),
                                 maximum_tokens=5)
    assert "".join(said) == generate(model, cfg.tokenizer, ["ACGTACGT"], maximum_tokens=5)[0]["text"]


def test_checkpoint_stores_posix_and_s3(tmp_path):
    """Uploads to a posix store (with retention) and to an S3 store driven through a fake client: retries, markers, and
    a failed upload that leaves `.uploading` in place so that pruning keeps the directory."""
    from savanna_b200.ckpt.io import _delete_old
    from savanna_b200.ckpt.stores import PosixStore, S3Store, upload_checkpoint
    root = tmp_path / "run"
    for step in (10, 20, 30):
        d = root / f"global_step{step}"
        (d / "configs").mkdir(parents=True)
        (d / "mp_rank_00_model_states.pt").write_bytes(b"x" * step)
        (d / "configs" / "a.yml").write_text("k: 1")

    class FakeS3:
        def __init__(self, fail_first=0, always_fail=False):
            self.calls, self.fail_first, self.always_fail, self.objects = 0, fail_first, always_fail, {}

        def upload_file(self, path, bucket, key):
            self.calls += 1
            if self.always_fail or self.calls <= self.fail_first:
                raise OSError("connection reset")
            self.objects[(bucket, key)] = open(path, "rb").read()

    naps = []
    posix = PosixStore({"location": str(tmp_path / "mirror"), "num_checkpoints": 2})
    s3 = S3Store({"bucket": "b", "location": "runs/x", "max_retries": 2}, client=FakeS3(fail_first=1))
    for step in (10, 20, 30):
        assert upload_checkpoint(str(root / f"global_step{step}"), [posix, s3], sleep=naps.append)
        assert (root / f"global_step{step}" / ".uploaded").exists() and not (root / f"global_step{step}" / ".uploading").exists()
    assert sorted(os.listdir(tmp_path / "mirror")) == ["global_step20", "global_step30"]          # keep last 2
    assert s3.client.objects[("b", "runs/x/global_step30/configs/a.yml")] == b"k: 1"
    assert len(s3.client.objects) == 6 and naps == [10.0]                                         # one retry, one delay
    bad = S3Store({"bucket": "b", "location": "", "max_retries": 1}, client=FakeS3(always_fail=True))
    (root / "global_step40").mkdir()
    (root / "global_step40" / "f.pt").write_bytes(b"y")
    assert not upload_checkpoint(str(root / "global_step40"), [bad], sleep=naps.append)
    assert (root / "global_step40" / ".uploading").exists() and not (root / "global_step40" / ".uploaded").exists()
    (root / "global_step50").mkdir()
    _delete_old(str(root), 1)                                  # would remove 10..40; 40 is still being uploaded
    assert sorted(p for p in os.listdir(root)) == ["global_step40", "global_step50"]


def test_zero3_layout_round_trips(tmp_path):
    """Stage-1 checkpoint -> stage-3 layout at dp=3 (a size that does not divide the parameters) -> re-partitioned to
    dp=2 -> back to stage 1: master weights and Adam moments survive bit for bit, the files carry the stage-3 keys, and
    the converted checkpoint loads into a trainer that continues the original loss trace."""
    from savanna_b200.ckpt import save_checkpoint
    from savanna_b200.tools import convert_zero3 as z3
    cfg = GlobalConfig.from_ymls([TINY], {"global_num_gpus": 1, "save": str(tmp_path / "ck"), "hidden_dropout": 0.0})
    tr = Trainer(cfg, load=False)

    def it(start=0):
        i = start
        while True:
            yield {"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i)}
            i += 1
    d = it()
    for _ in range(2):
        tr.train_step(d)
    src = save_checkpoint(tr)
    want_next = float(tr.train_step(d))
    s3, s3b, s1 = str(tmp_path / "z3" / "global_step2"), str(tmp_path / "z3b" / "global_step2"), str(tmp_path / "z1" / "global_step2")
    z3.from_zero1(src, s3, 3)
    names = sorted(os.listdir(s3))
    assert "zero_pp_rank_2_mp_rank_00_model_states.pt" in names and "zero_pp_rank_2_mp_rank_00_optim_states.pt" in names
    o = torch.load(os.path.join(s3, "zero_pp_rank_1_mp_rank_00_optim_states.pt"), weights_only=False)["optimizer_state_dict"]
    assert o["zero_stage"] == 3 and o["partition_count"] == 3 and "fp32_flat_groups" in o
    shapes = torch.load(os.path.join(s3, "zero_pp_rank_0_mp_rank_00_model_states.pt"), weights_only=False)["param_shapes"]
    want = sum(z3.partition_size(int(torch.Size(s).numel()), 3) for s in shapes[0].values())
    assert o["fp32_flat_groups"][0].numel() == want                       # every parameter cut on its own
    z3.repartition(s3, s3b, 2)
    z3.to_zero1(s3b, s1, 1)
    a = torch.load(os.path.join(src, "zero_pp_rank_0_mp_rank_00_optim_states.pt"), weights_only=False)["optimizer_state_dict"]
    b = torch.load(os.path.join(s1, "zero_pp_rank_0_mp_rank_00_optim_states.pt"), weights_only=False)["optimizer_state_dict"]
    for g in range(len(a["single_partition_of_fp32_groups"])):
        assert torch.equal(a["single_partition_of_fp32_groups"][g], b["single_partition_of_fp32_groups"][g])
        for key in ("exp_avg", "exp_avg_sq"):
            assert torch.equal(a["base_optimizer_state"]["state"][g][key], b["base_optimizer_state"]["state"][g][key])
    z3.to_fp32(s3, str(tmp_path / "w.pt"))
    w = torch.load(str(tmp_path / "w.pt"), weights_only=False)
    some = next(n for n in w if n.endswith("dense_projection.weight"))
    assert w[some].dtype == torch.float32 and w[some].shape == dict(tr.model.named_parameters())[some].shape
    with open(os.path.join(str(tmp_path / "z1"), "latest"), "w") as fh:
        fh.write("global_step2")
    cfg2 = GlobalConfig.from_ymls([TINY], {"global_num_gpus": 1, "load": str(tmp_path / "z1"), "hidden_dropout": 0.0})
    t2 = Trainer(cfg2, load=True)
    assert t2.iteration == 2
    assert abs(float(t2.train_step(it(2))) - want_next) < 1e-6


def test_train_tokenizer_round_trip(tmp_path):
    """A BPE tokenizer trained on a few jsonl lines loads through the framework's HFTokenizer and round-trips text."""
    import json
    pytest.importorskip("tokenizers")
    from savanna_b200.data.tokenizer import HFTokenizer
    from savanna_b200.tools import train_tokenizer as tt
    d = tmp_path / "corpus"
    d.mkdir()
    with open(d / "a.jsonl", "w") as fh:
        for i in range(50):
            fh.write(json.dumps({"text": f"the quick brown fox number {i} jumps over the lazy dog"}) + "\n")
    out = str(tmp_path / "tok" / "tok.json")
    tt.main(["--json_input_dir", str(d), "--tokenizer_output_path", out, "-v", "300"])
    tok = HFTokenizer(out)
    assert tok.eod == 0 and tok.pad_id == 1 and tok.vocab_size <= 300
    ids = tok.tokenize("the quick brown fox")
    assert tok.detokenize(ids).strip() == "the quick brown fox"
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError):
        list(tt.iter_texts(str(tmp_path / "empty")))


def test_modal_distillation_recovers_a_modal_filter():
    """Distilling a filter that is itself a sum of decaying modes: the real form reaches a small relative error and
    exports parameters that the framework's modal filter statement reproduces."""
    from savanna_b200.ops import reference as ref
    from savanna_b200.tools import distill_filters as df
    torch.manual_seed(0)
    N, O, L = 3, 4, 96
    gamma = torch.log(torch.rand(N, O) * 0.3 + 0.05)
    R = torch.randn(N, O) * 0.3
    p = -torch.ones(N, O)
    target = ref.modal_filter(gamma, R, p, L)
    models, logs = df.distill(target, order=8, form="real", epochs=1500, lr=2e-2)
    assert logs[0][-1] < logs[0][0] * 0.05
    err = df.relative_error(models[0], target)
    assert err < 0.15, err
    ex = df.export_implicit_modal(models[0])
    again = ref.modal_filter(ex["gamma"], ex["R"], ex["p"], L)
    assert torch.allclose(again, models[0].filter(L), atol=1e-5)
    # the complex (recurrent) form keeps tap 0 as a pass-through and fits the rest
    cm, clog = df.distill(target, order=8, form="complex", epochs=300, lr=1e-2)
    assert torch.allclose(cm[0].filter(L)[:, 0], target[:, 0]) and clog[0][-1] < clog[0][0]
    lam, Rc = cm[0].step_matrices()
    assert lam.shape == (N, 8) and Rc.is_complex()


def test_longeval_lines_task_scores_through_generation(tmp_path, monkeypatch):
    """LongEval plumbing with a stand-in generator: test files are written and read back, answers are parsed as the last
    integer, responses and accuracy land in the response file."""
    from savanna_b200.inference import longeval as le
    paths = le.write_testcases(str(tmp_path), "lines", sizes=[20, 30], num_cases=4, seed=1)
    assert len(paths) == 2 and all(os.path.exists(p) for p in paths)
    cases = le.load_testcases(paths[0])
    assert len(cases) == 4 and cases[0]["correct_line"].endswith(f"<{cases[0]['expected_number']}>")
    assert cases[0]["prompt"].count("REGISTER_CONTENT is") == 20
    assert le.parse_number("the value is <123> or 456") == 456 and le.parse_number("none") == -1
    answers = iter([f"it is {c['expected_number']}" if i % 2 == 0 else "unknown" for i, c in enumerate(cases)])
    monkeypatch.setattr(le, "_answer", lambda model, tok, prompt, n, cache: (next(answers), len(prompt)))
    out = str(tmp_path / "pred")
    os.makedirs(out)
    res = le.longeval_test(None, None, out, "lines", str(tmp_path), eval_shortest_only=True, sizes=[20, 30])
    assert list(res) == [20] and res[20]["accuracy"] == 0.5
    text = open(os.path.join(out, "20_response.txt")).read()
    assert text.count("Label:") == 4 and text.rstrip().endswith("Accuracy: 0.5")
    tp = le.write_testcases(str(tmp_path), "topics", sizes=[5], num_cases=2)
    tc = le.load_testcases(tp[0])
    assert len(tc[0]["topics"]) == 5 and tc[0]["topics"][0] in tc[0]["prompt"]


def test_prepare_dataset_from_local_files_and_upload_to_a_posix_store(tmp_path):
    """Corpora plumbing without network: a `file://` source is fetched, tokenised into .bin/.idx and read back; an
    unreachable URL gives a clear error; the upload tool copies a directory into a posix store with its marker."""
    from savanna_b200.data.indexed_dataset import make_dataset
    from savanna_b200.tools import corpora, prepare_data, upload
    src = tmp_path / "src.jsonl"
    with open(src, "w") as fh:
        for t in ("ACGTACGT", "GGCC", "TTTTAAAA"):
            fh.write(json.dumps({"text": t}) + "\n")
    prefix = prepare_data.main(["mygenomes", "-t", "CharLevelTokenizer", "-d", str(tmp_path / "data"), "--files", str(src),
                                "--workers", "1"])
    assert prefix.endswith(os.path.join("mygenomes", "mygenomes"))
    found = [p for p in os.listdir(os.path.dirname(prefix)) if p.endswith(".idx")]
    assert found, os.listdir(os.path.dirname(prefix))
    ds = make_dataset(os.path.join(os.path.dirname(prefix), found[0][:-4]))
    assert len(ds) == 3 and bytes(ds[1][:4].astype("uint8")) == b"GGCC"
    assert corpora.prepare_dataset("pass") is None
    with pytest.raises(NotImplementedError):
        corpora.prepare_dataset("no_such_corpus", "CharLevelTokenizer", str(tmp_path / "data"))
    with pytest.raises(RuntimeError, match="cannot download"):
        corpora.fetch("file:///nonexistent/file.jsonl", str(tmp_path / "x.jsonl"))
    ck = tmp_path / "global_step7"
    ck.mkdir()
    (ck / "mp_rank_00_model_states.pt").write_bytes(b"abc")
    assert upload.main(["store", str(ck), "--store", "posix", "--root", str(tmp_path / "archive")])
    assert (tmp_path / "archive" / "global_step7" / "mp_rank_00_model_states.pt").read_bytes() == b"abc"
    assert (ck / ".uploaded").exists()
