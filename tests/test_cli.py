"""The command line's options: the reference's names and older spellings
(src/support/options.cc:47-174), and what is refused because this engine does not have it.
No device is needed: refusals come before anything is loaded."""
import json

from inferx_b200.engine import cli


def test_reference_spellings_and_their_older_forms():
    p = cli.build_parser()
    a = p.parse_args(["folder", "--max-num-seqs", "3", "--max-model-len", "77",
                      "--num-gpu-blocks-override", "9", "--enforce-eager"])
    b = p.parse_args(["--model", "folder", "--max-running", "3", "--max-seq-len", "77",
                      "--kv-blocks", "9", "--no-cuda-graphs"])
    for args in (a, b):
        assert (args.max_num_seqs, args.max_model_len, args.num_gpu_blocks_override,
                args.enforce_eager) == (3, 77, 9, True)
    assert a.model_pos == "folder" and b.model == "folder"
    d = p.parse_args(["folder"])
    assert (d.dtype, d.block_size, d.gpu_memory_utilization, d.enforce_eager,
            d.chunked_prefill, d.prefix_caching, d.log_level) == \
        ("auto", 16, 0.92, False, True, False, "info")
    s = p.parse_args(["folder", "--presence-penalty", "0.5", "--frequency-penalty", "0.25",
                      "--repetition-penalty", "1.2", "--min-tokens", "4", "--logprobs", "3",
                      "--top-k", "5", "--top-p", "0.9", "--min-p", "0.1", "--temperature", "0.7"])
    assert (s.presence_penalty, s.frequency_penalty, s.repetition_penalty, s.min_tokens,
            s.logprobs, s.top_k, s.top_p, s.min_p, s.temperature) == \
        (0.5, 0.25, 1.2, 4, 3, 5, 0.9, 0.1, 0.7)
    assert p.parse_args(["folder"]).logprobs is None


def test_what_this_engine_does_not_have_is_refused_with_the_reason(capsys):
    base = ["folder", "--prompt-ids", "1,2"]
    for extra, word in ((["--dtype", "half"], "bfloat16 or float32"),
                        (["--no-enable-chunked-prefill"], "cannot be disabled"),
                        (["--enable-prefix-caching"], "no prefix cache"),
                        (["--tensor-parallel-size", "2"], "one GPU"),
                        (["--device", "rocm"], "CUDA only"),
                        (["-q", "fp8"], "bfloat16 or float32"),
                        (["--kv-cache-dtype", "fp8"], "element type")):
        assert cli.main(base + extra) == 2
        assert word in capsys.readouterr().err
    # the values that mean "off" pass this stage (and then stop for want of prompts)
    assert cli.main(["folder", "--no-enable-prefix-caching", "--enable-chunked-prefill",
                     "--tensor-parallel-size", "1", "--device", "cuda", "--kv-cache-dtype",
                     "auto", "--no-enforce-eager"]) == 2
    assert "no prompts" in capsys.readouterr().err


def test_log_lines_plain_json_and_to_a_file(tmp_path, capsys):
    path = tmp_path / "log.txt"
    log = cli._Log("info", True, str(path))
    log("debug", "not shown")
    log("info", "model ready", cache_pages=[32])
    log("warning", "careful")
    err = capsys.readouterr().err.splitlines()
    recs = [json.loads(ln) for ln in err]
    assert [r["msg"] for r in recs] == ["model ready", "careful"]
    assert recs[0]["level"] == "info" and recs[0]["cache_pages"] == [32]
    assert path.read_text().splitlines() == err
    cli._Log("warning", False, None)("error", "plain", steps=3)
    assert capsys.readouterr().err.strip() == "[inferx-generate] plain steps=3"
