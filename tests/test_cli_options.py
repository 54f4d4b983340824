"""The command line's options: the reference's names and defaults where it has them
(crates/synaptix-cli/src/bin/synaptix.rs:49-135, `Run` and `Bench`)."""
import pytest

from synaptix_b200 import cli, ops


def test_run_and_bench_take_the_references_options_with_its_defaults():
    p = cli.build_parser()
    a = p.parse_args(["run", "MODEL"])
    assert (a.prompt, a.max_tokens, a.temperature, a.seed, a.device, a.max_seq, a.attn) == ("", 128, 1.0, 0, "cuda", None, None)
    assert (a.prompt_file, a.no_graph, a.warmup, a.prefill_batch) == (None, False, False, 0)
    a = p.parse_args(["run", "MODEL", "5 17 3", "--max-tokens", "9", "--temperature", "0", "--top-k", "40", "--top-p", "0.9",
                      "--min-p", "0.05", "--repetition-penalty", "1.1", "--seed", "7", "--max-seq", "512", "--attn", "fa2",
                      "--compute-dtype", "f32", "--no-graph", "--warmup", "--prefill-batch", "256"])
    assert (a.max_tokens, a.top_k, a.top_p, a.min_p, a.repetition_penalty, a.prefill_batch) == (9, 40, 0.9, 0.05, 1.1, 256)
    b = p.parse_args(["bench", "MODEL"])
    assert (b.n_tokens, b.prompt_tokens, b.batch_size, b.warmup, b.device, b.attn) == (128, 0, 1, 3, "cuda", None)


def test_attn_names_choose_the_prompt_attention_kernel():
    was = ops.OPTIONS.attn_tc
    try:
        for name, want in (("fa2", False), ("fa4", True), ("flash-attn-2", False), ("FA4", True)):
            cli._set_attn(name)
            assert ops.OPTIONS.attn_tc is want
        ops.set_options(attn_tc=False)
        for name in (None, "auto", "flash-decode", "decode"):       # leave the choice as it is
            cli._set_attn(name)
            assert ops.OPTIONS.attn_tc is False
        with pytest.raises(SystemExit):
            cli._set_attn("fa3")
    finally:
        ops.set_options(attn_tc=was)


def test_inspect_lists_a_model_folder(tmp_path, capsys):
    """``inspect`` (the reference has the command for safetensors files, commands/inspect.rs:66-93), on the CPU."""
    import tiny
    folder = tiny.make_folder("A", str(tmp_path / "a"))
    assert cli.main(["inspect", folder]) == 0
    out = capsys.readouterr().out
    assert "architecture: Qwen3ForCausalLM (qwen3)" in out and "hidden_size: 64" in out
    assert "cache, bfloat16: 256 bytes a token" in out                    # 2 layers x 2 kv heads x 16 x (K and V) x 2 bytes
    assert "model.layers.1.self_attn.q_norm.weight" in out and "model.embed_tokens.weight" in out
    n = 2 * 11 + 2                                                         # 11 tensors a layer, embedding and final norm (tied head)
    assert f"shown {n} of {n} tensors" in out
    assert cli.main(["inspect", folder + "/model.safetensors", "-f", "layers.0.mlp", "-v"]) == 0
    out = capsys.readouterr().out
    assert f"shown 3 of {n} tensors" in out and "bytes=" in out and "layers.1" not in out.split("total tensors")[1].split("shown")[0]
