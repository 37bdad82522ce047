"""The command line: option names as the reference's, `info` without torch-side work."""

from __future__ import annotations

import json

import pytest

from inference_engine_b200 import cli
from tests import helpers as H
from tests.tiny_configs import TINY_B


def test_info_prints_the_shape(tmp_path, capsys):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert cli.main(["info", "--model", str(tmp_path), "--gpu-mem", "180"]) == 0
    out = capsys.readouterr().out
    assert "architecture        LlamaForCausalLM" in out
    assert "layers / hidden     3 / 96" in out
    assert "heads (q / kv)      3 / 1  (GQA groups: 3, head dim 32)" in out
    assert "On a 180 GiB GPU" in out and "KV tokens fit" in out


def test_generate_options_are_the_references():
    args = cli.build_parser().parse_args(["generate", "--model", "m", "--prompt", "hi"])
    assert (args.temperature, args.top_p, args.max_tokens, args.seed, args.device) == (0.7, 0.9, 256, None, "cuda")
    assert (args.max_num_seqs, args.max_num_batched_tokens, args.block_size, args.num_blocks) == (64, 4096, 16, None)
    assert args.gpu_memory_utilization == 0.9 and not args.no_chunked_prefill and not args.no_cuda_graphs
    with pytest.raises(SystemExit):
        cli.build_parser().parse_args(["serve", "--model", "m"])  # there is no server


@pytest.mark.gpu
def test_generate_runs_from_a_folder(tmp_path, capsys):
    folder = H.write_model_dir(tmp_path / "m", TINY_B, H.make_weights(TINY_B, seed=1))
    rc = cli.main(["generate", "--model", str(folder), "--prompt-ids", "5,17,3,99", "--temperature", "0",
                   "--max-tokens", "5", "--dtype", "float32", "--num-blocks", "16", "--block-size", "8",
                   "--max-num-seqs", "2", "--max-num-batched-tokens", "64"])
    assert rc == 0
    from tests import plain_llama

    want = plain_llama.greedy_generate(TINY_B, H.make_weights(TINY_B, seed=1), [5, 17, 3, 99], 5,
                                       stop_ids=(2, 3))
    captured = capsys.readouterr()
    assert captured.out.split() == [str(t) for t in want]
    assert "tokens/s" in captured.err


def test_info_prints_a_rugedra_shape(tmp_path, capsys):
    from tests import rugedra_configs as R

    (tmp_path / "config.json").write_text(json.dumps(R.with_ranks(R.MIXED)))
    assert cli.main(["info", "--model", str(tmp_path), "--gpu-mem", "180"]) == 0
    out = capsys.readouterr().out
    assert "architecture        Rugedra" in out and "layers / width      4 / 72" in out
    assert "channel_delta+moe, latent_attention, latent_attention+dense, channel_delta+dense" in out
    assert "state per request" in out


def test_info_prints_a_ravapel_shape(tmp_path, capsys):
    from tests import ravapel_configs as R

    (tmp_path / "config.json").write_text(json.dumps(R.MIXED))
    assert cli.main(["info", "--model", str(tmp_path), "--gpu-mem", "180"]) == 0
    out = capsys.readouterr().out
    assert "architecture        Ravapel" in out and "layers / width      5 / 72" in out
    assert "hgrn2+dense, parallel, hgrn2+dense, parallel+dense, hgrn2+dense" in out
    assert "loop                layers 1..2 x 3" in out and "state per request" in out


@pytest.mark.gpu
def test_generate_runs_a_ravapel_folder(tmp_path, capsys):
    """`engine generate` on a Ravapel folder: the same entry point, scheduler and sampling as for the
    other architectures; greedy tokens are the plain implementation's."""
    import torch

    from tests import plain_ravapel as P
    from tests import ravapel_configs as R

    cfg, weights = R.ODD, R.make_weights(R.ODD, seed=2)
    folder = H.write_model_dir(tmp_path / "m", cfg, weights)
    prompt = [5, 17, 3, 44, 9, 21, 30]
    rc = cli.main(["generate", "--model", str(folder), "--prompt-ids", ",".join(map(str, prompt)), "--temperature", "0",
                   "--max-tokens", "6", "--dtype", "float32", "--num-blocks", "16", "--block-size", "8",
                   "--max-num-seqs", "2", "--max-num-batched-tokens", "4"])
    assert rc == 0
    ids = list(prompt)
    for _ in range(6):
        ids.append(int(P.forward(cfg, weights, ids, torch.float64)[-1].argmax()))
    assert capsys.readouterr().out.split() == [str(t) for t in ids[len(prompt):]]


def test_info_prints_a_vofanex_shape(tmp_path, capsys):
    from tests import vofanex_configs as V

    folder = H.write_model_dir(tmp_path / "m", V.MIXED, V.make_weights(V.MIXED, seed=2))
    assert cli.main(["info", "--model", str(folder), "--gpu-mem", "180"]) == 0
    out = capsys.readouterr().out
    assert "architecture        Vofanex" in out and "layers / width      5 / 72" in out
    assert "gla+dense, attention+moe, gla, attention+dense, gla+moe" in out
    assert "attention windows   7, 10" in out and "state per request" in out


@pytest.mark.gpu
def test_generate_runs_a_vofanex_folder(tmp_path, capsys):
    """`engine generate` on a Vofanex folder: the same entry point, scheduler and sampling as for the
    other architectures; greedy tokens are the plain implementation's."""
    import torch

    from tests import plain_vofanex as P
    from tests import vofanex_configs as V

    cfg, weights = V.ODD, V.make_weights(V.ODD, seed=2)
    folder = H.write_model_dir(tmp_path / "m", cfg, weights)
    prompt = [5, 17, 3, 44, 9, 21, 30]
    rc = cli.main(["generate", "--model", str(folder), "--prompt-ids", ",".join(map(str, prompt)), "--temperature", "0",
                   "--max-tokens", "6", "--dtype", "float32", "--num-blocks", "16", "--block-size", "8",
                   "--max-num-seqs", "2", "--max-num-batched-tokens", "4"])
    assert rc == 0
    ids = list(prompt)
    for _ in range(6):
        ids.append(int(P.forward(cfg, weights, ids, torch.float64)[-1].argmax()))
    assert capsys.readouterr().out.split() == [str(t) for t in ids[len(prompt):]]


def test_info_prints_a_puposun_shape(tmp_path, capsys):
    from tests import puposun_configs as V

    folder = H.write_model_dir(tmp_path / "m", V.MIXED, V.make_weights(V.MIXED, seed=2))
    assert cli.main(["info", "--model", str(folder), "--gpu-mem", "180"]) == 0
    out = capsys.readouterr().out
    assert "architecture        Puposun" in out and "layers / width      4 / 72" in out
    assert "attention+moe, attention_2+moe, attention_2, attention+moe" in out
    assert "loop                layers 1..2 x 2" in out and "attention windows   7 (+ first 0), 10 (+ first 3)" in out


@pytest.mark.gpu
def test_generate_runs_a_puposun_folder(tmp_path, capsys):
    """`engine generate` on a Puposun folder: the same entry point, scheduler and sampling as for the
    other architectures; greedy tokens are the plain implementation's."""
    import torch

    from tests import plain_puposun as P
    from tests import puposun_configs as V

    cfg, weights = V.MIXED, V.make_weights(V.MIXED, seed=2)
    folder = H.write_model_dir(tmp_path / "m", cfg, weights)
    prompt = [5, 17, 3, 44, 9, 21, 30, 8, 100, 61, 2, 77, 13]
    rc = cli.main(["generate", "--model", str(folder), "--prompt-ids", ",".join(map(str, prompt)), "--temperature", "0",
                   "--max-tokens", "6", "--dtype", "float32", "--num-blocks", "16", "--block-size", "8",
                   "--max-num-seqs", "2", "--max-num-batched-tokens", "4"])
    assert rc == 0
    ids = list(prompt)
    for _ in range(6):
        ids.append(int(P.forward(cfg, weights, ids, torch.float64)[-1].argmax()))
    assert capsys.readouterr().out.split() == [str(t) for t in ids[len(prompt):]]
