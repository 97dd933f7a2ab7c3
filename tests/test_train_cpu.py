

def test_mup_coord_check(tmp_path):
    """Three widths, with and without muP: every block is recorded at every step; the CSV and the slopes come out."""
    import os
    from savanna_b200.train import mup_coord_check as cc
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tiny = os.path.join(root, "configs", "baseline", "tiny_sh2_cpu.yml")
    recs = cc.coord_check([tiny], {"global_num_gpus": 1, "seq_length": 64, "max_position_embeddings": 64,
                                   "train_micro_batch_size_per_gpu": 1, "gradient_accumulation_steps": 1},
                          powers=[2, 3, 4], steps=2)
    widths = sorted({r["width"] for r in recs})
    assert len(widths) == 3 and widths[1] == 2 * widths[0]
    assert {r["mup"] for r in recs} == {0, 1} and {r["step"] for r in recs} == {0, 1}
    assert {"embedding", "block0", "logits"} <= {r["module"] for r in recs}
    cc.write_csv(recs, str(tmp_path / "cc.csv"))
    assert len(open(tmp_path / "cc.csv").read().splitlines()) == len(recs) + 1
    s = cc.summarise(recs)
    assert set(s) == {"mup", "sp"} and "logits" in s["mup"] and all(v == v for v in s["sp"].values())
