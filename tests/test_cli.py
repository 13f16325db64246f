"""The package's inspection commands (no GPU needed for list / show / source)."""

from mlc_compiler_b200.__main__ import main


def test_list_show_and_source(capsys):
    assert main(["list"]) == 0
    assert "bert-base_b1_s128_float16" in capsys.readouterr().out
    assert main(["show", "gpt2-small_b1_s128_float16"]) == 0
    out = capsys.readouterr().out
    assert "schedule(148 kernels" in out and "memory: arena 1920.0 KiB" in out
    assert main(["source", "bert-base_b1_s128_float16", "--kernel", "k13"]) == 0
    out = capsys.readouterr().out
    assert 'extern "C" __global__' in out and "k13" in out and "persistent" in out


def test_source_of_an_extern_kernel_is_refused(capsys):
    assert main(["source", "bert-base_b1_s128_float16", "--kernel", "k6"]) == 1
    assert "extern kernel" in capsys.readouterr().err
    assert main(["source", "bert-base_b1_s128_float16", "--kernel", "k9999"]) == 1
    assert "no kernel named" in capsys.readouterr().err


def test_rewritten_view_shows_forwarded_producers(capsys):
    assert main(["show", "bert-base_b8_s128_float16", "--rewritten"]) == 0
    out = capsys.readouterr().out
    assert "schedule(184 kernels" in out and "clone" not in out and "[embedding, embedding" in out
