"""Real-weights workflow (esmm-research_b200/real_weights.py): the host-side helpers follow the
reference's tests/test_benchmark_ab_real.py; the GPU test runs both modes on small stored matrices."""
import csv
import importlib.util
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def rw(pkg):
    spec = importlib.util.spec_from_file_location("esmm_real_weights",
                                                  os.path.join(ROOT, "esmm-research_b200", "real_weights.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_pad_to_tile(rw):
    arr = np.ones((64, 16), np.float32)
    assert rw.pad_to_tile(arr) is arr
    out = rw.pad_to_tile(np.ones((33, 9), np.float32))
    assert out.shape == (64, 16) and out[33, 9] == 0.0 and out[0, 0] == 1.0 and out[32, 8] == 1.0
    assert rw.pad_to_tile(np.ones((9, 33), np.float32), rw.BK, rw.BM).shape == (16, 64)


def test_compute_block_sparsity(rw):
    assert rw.compute_block_sparsity(np.ones((64, 16), np.float32)) == 0.0
    assert rw.compute_block_sparsity(np.zeros((64, 16), np.float32)) == 1.0
    arr = np.zeros((64, 16), np.float32)
    arr[:32, :] = 1.0
    assert rw.compute_block_sparsity(arr) == pytest.approx(0.5)
    arr[40, 9] = -0.0  # negative zero does not make a tile live
    assert rw.compute_block_sparsity(arr) == pytest.approx(0.5)


def _save(tmp_path, name, shape, kind="pt"):
    p = tmp_path / name
    if kind == "pt":
        import torch
        torch.save(torch.zeros(shape), p)
    elif kind == "npy":
        np.save(p, np.zeros(shape, np.float32))
    else:
        np.zeros(shape, np.float32).tofile(p)
    return p


def test_find_compatible_pairs(rw, tmp_path):
    a = _save(tmp_path, "a_permuted.pt", (128, 256))
    b = _save(tmp_path, "b_permuted.pt", (256, 64))
    c = _save(tmp_path, "c_permuted.pt", (64, 256))          # rows 64 != A's 256 columns
    logs = []
    assert rw.find_compatible_pairs([a], [b], log=logs.append) == [(a, b)]
    assert rw.find_compatible_pairs([a], [c], log=logs.append) == []
    assert rw.find_compatible_pairs([a], [a], log=logs.append) == []           # same file on both sides
    assert rw.find_compatible_pairs([a], [b], max_k=128, log=logs.append) == []
    assert any("K=256 > 128" in m for m in logs)
    # other containers, and unreadable ones skipped with a reason
    n = _save(tmp_path, "w.npy", (256, 96), "npy")
    r = _save(tmp_path, "w_256x32.bin", (256, 32), "bin")
    bad = _save(tmp_path, "w_256x64.bin", (256, 32), "bin")
    v = tmp_path / "vec_permuted.pt"
    import torch
    torch.save(torch.zeros(7), v)
    assert rw.find_compatible_pairs([a], [n, r, bad, v], log=logs.append) == [(a, n), (a, r)]
    assert any("file size does not match" in m for m in logs) and any("not a 2D tensor" in m for m in logs)
    assert rw.matrix_shape(r)[0] == (256, 32) and rw.load_matrix(r).shape == (256, 32)
    assert [p.name for p in rw.find_weight_files(tmp_path, "w")] == ["w.npy", "w_256x32.bin", "w_256x64.bin"]


def test_parse_config_and_csv_columns(rw, tmp_path):
    p = tmp_path / "wanda" / "grp_8" / "col_perm" / "sparsity_0.99" / "layer3_permuted.pt"
    assert rw.parse_config(p) == {"pruner": "wanda", "group_size": "8", "perm_type": "col", "sparsity": "0.99"}
    q = tmp_path / "sparsegpt" / "grp_16_rows_permuted" / "sparsity_0.5" / "x.pt"
    assert rw.parse_config(q) == {"pruner": "sparsegpt", "group_size": "16", "perm_type": "row", "sparsity": "0.5"}
    timings = {15: (2.0, 0.0), 29: (0.4, 0.1), 20: (None, None)}
    row = {"layer": "x"}
    rw.timing_columns(row, [15, 29, 20], timings)
    rw.speedup_columns(row, timings)
    assert row == {"layer": "x", "k15_compute_ms": "2.000", "k15_preprocess_ms": "0.000", "k29_compute_ms": "0.400",
                   "k29_preprocess_ms": "0.100", "k20_compute_ms": "N/A", "k20_preprocess_ms": "N/A",
                   "k29_compute_speedup": "5.000", "k29_total_speedup": "4.000"}
    rw.write_csv(tmp_path / "out" / "r.csv", [row])
    with open(tmp_path / "out" / "r.csv") as f:
        assert list(csv.DictReader(f))[0]["k29_total_speedup"] == "4.000"
    lines = rw.summary_lines([row])
    assert "1 rows" in lines[0] and "mean=5.00x" in lines[1] and "mean=4.00x" in lines[2]
    assert rw.main(["--weights", str(tmp_path / "nothing")]) == 1


@pytest.mark.gpu
def test_both_modes_on_stored_matrices(rw, cuda, tmp_path, capfd):
    import workloads
    import oracle
    A, B = workloads.tile_random(200, 352, 250, 0.5, 0.4, seed=5, gran_a=32, gran_b=32)   # ragged on purpose
    wdir = tmp_path / "wanda" / "sparsity_0.5"
    wdir.mkdir(parents=True)
    np.save(wdir / "act.npy", A)
    B.tofile(wdir / f"w_{B.shape[0]}x{B.shape[1]}.bin")
    out = tmp_path / "pairs.csv"
    assert rw.main(["--weights-a", str(wdir), "--weights-b", str(wdir), "--filter-a", "act", "--filter-b", "w_",
                    "--kernels", "15,29,20,21,129", "--runs", "2", "--out", str(out)]) == 0
    text = capfd.readouterr().out
    assert "B patterns: saved" in text and "FAILED" not in text
    with open(out) as f:
        rows = list(csv.DictReader(f))
    assert len(rows) == 1 and rows[0]["a_shape"] == "200x250" and rows[0]["b_shape"] == "250x352"
    assert float(rows[0]["k29_compute_ms"]) > 0 and float(rows[0]["k29_total_speedup"]) > 0
    assert float(rows[0]["k129_compute_ms"]) > 0          # the optional tensor-core variant, verified against cuBLAS too
    # the cache holds the oracle's bytes for the padded B, and the second run loads it
    raw = (wdir / f"w_{B.shape[0]}x{B.shape[1]}.bin.bpat").read_bytes()
    Bp = rw.pad_to_tile(B, rw.BK, rw.BM)
    assert np.array_equal(np.frombuffer(raw[32:], np.uint8).reshape(Bp.shape[1] // 32, Bp.shape[0] // 8),
                          oracle.preprocess_b(Bp))
    out2 = tmp_path / "single.csv"
    assert rw.main(["--weights", str(wdir), "--filter-b", "w_", "--rows", "256", "--runs", "2", "--out", str(out2)]) == 0
    text = capfd.readouterr().out
    assert "B patterns: loaded" in text and "K29 vs cuBLAS - 1 rows" in text
    with open(out2) as f:
        rows = list(csv.DictReader(f))
    assert rows[0]["orig_shape"] == "250x352" and rows[0]["sparsity"] == "0.5" and rows[0]["pruner"] == "wanda"
