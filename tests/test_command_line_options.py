"""The command line's options and prompt forms, without a GPU: names and defaults after the reference's
(src/main.c:188-340, 505-575)."""
import pytest

from xyntetik_runner_b200.cli import build_parser, encode_prompt, main, unescape


def test_option_names_and_defaults():
    a = build_parser().parse_args(["-m", "folder", "-p", "hi"])
    assert (a.n, a.temp, a.top_k, a.top_p, a.min_p, a.repeat_penalty) == (256, 0.0, 0, 1.0, 0.0, 1.0)
    assert a.seed is None and a.ctx is None and a.parallel == 1 and not a.ignore_eos and not a.no_bos and not a.score
    a = build_parser().parse_args(["-m", "f", "-p", "x", "-n", "-1", "-c", "512", "-b", "64", "-s", "7", "--temp", "0.6", "--top-k", "40",
                                   "--top-p", "0.9", "--min-p", "0.05", "--repeat-penalty", "1.1", "--ignore-eos", "--no-bos",
                                   "--score", "--parallel", "4", "--rope-base", "10000", "--rope-scale", "2", "--dtype", "float32"])
    assert (a.n, a.ctx, a.batch, a.seed, a.temp, a.top_k, a.parallel) == (-1, 512, 64, 7, 0.6, 40, 4)
    assert a.rope_base == 10000.0 and a.rope_scale == 2.0 and a.score and a.dtype == "float32"


def test_prompt_forms():
    assert unescape(r"a\nb\tc\\d\r") == "a\nb\tc\\d\r" and unescape("plain\\x") == "plain\\x"
    assert encode_prompt("ids:1, 5,9", 10) == [1, 5, 9]
    assert encode_prompt("AB", 256) == [65, 66] and encode_prompt("é", 256) == [0xC3, 0xA9]
    with pytest.raises(SystemExit, match="outside the vocabulary"):
        encode_prompt("ids:1,300", 256)
    with pytest.raises(SystemExit, match="comma-separated"):
        encode_prompt("ids:1,x", 256)


def test_refusals_before_anything_is_loaded(capsys):
    assert main(["-p", "x"]) == 2 and "-m MODEL is required" in capsys.readouterr().err
    assert main(["-m", "folder", "-p", "x", "-s", "0"]) == 2 and "refused" in capsys.readouterr().err


def test_ref_runs_the_plain_implementation_without_a_gpu(tmp_path, capsys):
    """--ref: greedy tokens of the plain implementation, from the same folder and prompt syntax as the engine's."""
    import tiny
    from plain_llama import PlainLlama
    folder = tiny.make_folder(str(tmp_path / "a"), "A")
    assert main(["-m", folder, "-p", "ids:7,8,9,200", "-n", "5", "--ref", "--ignore-eos", "-t", "2"]) == 0
    out = capsys.readouterr().out.strip()
    bos = tiny.TINY_A["bos_token_id"]
    assert out == "ids:" + ",".join(str(t) for t in PlainLlama(folder).generate_greedy([bos, 7, 8, 9, 200], 5))
    assert main(["-m", folder, "-p", "x", "--ref", "--temp", "0.5"]) == 2
