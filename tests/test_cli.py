"""The command line's parts that need no GPU: writing a random model folder from sizes, folding bench lines
into a table, and the messages for a missing model."""

import json

import pytest

from nanospec_b200.__main__ import fold_bench_lines, main


def test_random_weights_command_writes_a_folder_that_reads_back(tmp_path):
    out = tmp_path / "m"
    rc = main(["random-weights", "--out", str(out), "--seed", "4", "--vocab-size", "331", "--hidden-size", "96",
               "--intermediate-size", "200", "--num-hidden-layers", "2", "--num-attention-heads", "6",
               "--num-key-value-heads", "3", "--head-dim", "16", "--max-position-embeddings", "384"])
    assert rc == 0
    cfg = json.loads((out / "config.json").read_text())
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["vocab_size"] == 331 and cfg["num_key_value_heads"] == 3
    assert (out / "model.safetensors").stat().st_size > 0
    # the same seed gives the same bytes
    again = tmp_path / "m2"
    main(["random-weights", "--out", str(again), "--seed", "4", "--vocab-size", "331", "--hidden-size", "96",
          "--intermediate-size", "200", "--num-hidden-layers", "2", "--num-attention-heads", "6",
          "--num-key-value-heads", "3", "--head-dim", "16", "--max-position-embeddings", "384"])
    assert (out / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()


def test_table_takes_the_median_over_runs_and_skips_other_lines(tmp_path, capsys):
    rows = [dict(engine="nanospec_b200", config="nospec", bs=8, tok_s=t, tpot_ms=p, dtype="bfloat16", gpu="B200", run=i)
            for i, (t, p) in enumerate([(100.0, 10.0), (300.0, 12.0), (200.0, 11.0)])]
    rows.append(dict(engine="nanospec_b200", config="nospec", bs=1, tok_s=50.0, tpot_ms=None))
    text = fold_bench_lines(["[nanospec_b200] compiled x.cu\n"] + [json.dumps(r) + "\n" for r in rows])
    lines = text.splitlines()
    assert lines[0].startswith("| engine |") and len(lines) == 4
    assert lines[2] == "| nanospec_b200 | nospec | 1 | 50.0 | - | 1 | - | - |"       # batch sizes in ascending order
    assert lines[3] == "| nanospec_b200 | nospec | 8 | 200.0 | 11.0 | 3 | bfloat16 | B200 |"
    path = tmp_path / "lines.jsonl"
    path.write_text("".join(json.dumps(r) + "\n" for r in rows))
    assert main(["table", str(path)]) == 0
    assert capsys.readouterr().out.strip() == text


def test_a_command_without_a_model_says_so(monkeypatch):
    monkeypatch.delenv("NANOSPEC_MODEL", raising=False)
    with pytest.raises(SystemExit) as e:
        main(["generate", "--prompt-ids", "1,2,3"])
    assert str(e.value) == "no model folder: give --model or set NANOSPEC_MODEL"
