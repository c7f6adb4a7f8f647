"""The roofline report is generated from the benchmarks' JSON files; here from small hand-made ones."""
import json

from tips_b200.bench import roofline_report as R


def test_report_tables(tmp_path):
    kernels = {"peaks": {"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "source": "measured"},
               "results": [{"kernel": "gemm", "shape": [4096, 4096, 4096], "ms": 0.2, "tflops": 800.0,
                            "library_ms(linear+relu)": 0.1},
                           {"kernel": "adam", "elements": 1 << 20, "ms": 0.5, "gbs": 3250.0},
                           {"kernel": "conv", "hw": 56, "cin": 64, "cout": 64, "k": 3, "stride": 1, "gflop": 100.0,
                            "fwd_ms": 0.1, "fwd_lib_ms": 0.05, "fwd_tflops": 1000.0,
                            "dgrad_ms": 0.2, "dgrad_lib_ms": 0.4, "wgrad_ms": 0.25, "wgrad_lib_ms": 0.25},
                           {"conv_total_ms": {"fwd": 1.0}}]}
    sweep = {"ranks": 8, "uses_multimem": True,
             "rows": [{"dtype": "bf16", "bytes": 1 << 26, "ranks": 8, "allreduce_inplace_ms": 0.2,
                       "allreduce_inplace_busbw": 587.2, "nccl_allreduce_busbw": 400.0, "allgather_busbw": 500.0,
                       "nccl_allgather_busbw": 550.0, "broadcast_gbs": 300.0}]}
    bench = {"n_gpus": 1, "metric": "resnet50_train_images_per_sec", "value": 10000.0, "unit": "images/s",
             "ms_per_step": 25.6, "e2e": {"value": 9900.0}, "floor": {"resnet50": {"value": 5000.0}, "ps": {"value": 5e6}},
             "vs_floor": {"resnet50": 2.0, "ps": 4.0},
             "ps": {"metric": "ps_ctr_train_samples_per_sec", "value": 2e7, "unit": "samples/s", "ms_per_step": 0.4,
                    "e2e": {"value": 1.9e7}}}
    rows, src, _ = R.kernel_rows(kernels)
    assert src == "measured" and len(rows) == 5
    gemm = rows[0]
    assert gemm[0] == "gemm" and abs(gemm[5] - 0.5) < 1e-9 and abs(gemm[7] - 0.5) < 1e-9
    assert abs(rows[1][5] - 0.5) < 1e-9                      # 3250 of 6500 GB/s
    conv = {r[0]: r for r in rows[2:]}
    assert abs(conv["conv fwd"][5] - 1000.0 / 1600.0) < 1e-9
    assert abs(conv["conv dgrad"][3] - 0.5) < 1e-9           # 100 GFLOP in 0.2 ms
    assert abs(conv["conv dgrad"][7] - 2.0) < 1e-9
    n, srows = R.sweep_rows(sweep)
    assert n == 8 and abs(srows[0][3] - ((1 << 26) * 9 / 8 / 770e6) / 0.2) < 1e-9
    brows = R.bench_rows(bench)
    assert [b[0] for b in brows] == ["resnet50_train_images_per_sec", "ps_ctr_train_samples_per_sec"]
    assert brows[0][7] == 2.0 and brows[1][6] == 5e6
    paths = []
    for name, doc in (("k.json", kernels), ("s.json", sweep), ("b.json", bench)):
        p = tmp_path / name
        p.write_text(("log line\n" if name == "b.json" else "") + json.dumps(doc))
        paths.append(str(p))
    out = tmp_path / "report.md"
    R.main(["--kernels", paths[0], "--sweep", paths[1], "--bench", paths[2], "--out", str(out)])
    text = out.read_text()
    assert "of measured peak" in text and "Collectives on 8 GPUs" in text and "| 2x |" in text
    assert "conv dgrad | 56x56 64->64 k3 s1" in text
