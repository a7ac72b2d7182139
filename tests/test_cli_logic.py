"""The command line's own logic (arguments, what is printed in which form, errors), run inside
this process on the torch-CPU stand-in of the kernel library.  The program as a user runs it,
on the GPU, is in test_gpu_generate.py."""
import json

import pytest
import torch

import plain_gpt2 as P
from nimbus_infer_rs_b200.__main__ import _parse_ids, main

CPU = ["--device", "cpu", "--dtype", "float32"]


def test_id_lists():                                   # src/main.rs:130-134, `;` between requests
    assert _parse_ids("1,2,3") == [[1, 2, 3]]
    assert _parse_ids(" 5 , 17;9 ;") == [[5, 17], [9]]
    for bad in ("", ";", "1,x"):
        with pytest.raises(SystemExit):
            _parse_ids(bad)


def test_generate_one_request_and_several(model_dirs, cpu_backend, capsys):
    W = P.PlainWeights(model_dirs["A"])
    want = P.greedy_generate(W, [5, 17, 3], 5)
    assert main(["generate", "--model", str(model_dirs["A"]), "--ids", "5,17,3",
                 "--max-new-tokens", "5", "--json", *CPU]) == 0
    io = capsys.readouterr()
    assert json.loads(io.out) == {"prompt_tokens": 3, "generated_ids": want, "text": str(want)}
    assert "tok/s]" in io.err                          # src/main.rs:186
    # several requests, streamed: `request:token` as they come, then a list a request
    want2 = P.greedy_generate(W, [9], 5)
    assert main(["generate", "--model", str(model_dirs["A"]), "--ids", "5,17,3;9",
                 "--max-new-tokens", "5", "--stream", *CPU]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    streamed = [tuple(int(x) for x in item.split(":")) for item in lines[0].split()]
    assert [t for r, t in streamed if r == 0] == want and [t for r, t in streamed if r == 1] == want2
    assert [json.loads(l) for l in lines[1:]] == [want, want2]
    # a stop token ends the request with it; temperature 0 is the command line's default
    assert main(["generate", "--model", str(model_dirs["A"]), "--ids", "5,17,3", "--stop",
                 str(want[2]), "--json", *CPU]) == 0
    assert json.loads(capsys.readouterr().out)["generated_ids"] == want[:want.index(want[2]) + 1]


def test_sampling_options_reach_the_sampler(cpu_backend, capsys):
    args = ["generate", "--random", "tiny-b", "--seed-weights", "2", "--ids", "5,17,3",
            "--max-new-tokens", "6", "--json", *CPU]
    def ids(*more):
        assert main([*args, *more]) == 0
        return json.loads(capsys.readouterr().out)["generated_ids"]
    greedy = ids()
    assert ids("--temperature", "5.0", "--top-k", "1", "--seed", "4") == greedy
    assert ids("--temperature", "5.0", "--top-p", "0.0", "--seed", "4") == greedy
    hot = ids("--temperature", "5.0", "--seed", "4")
    assert hot == ids("--temperature", "5.0", "--seed", "4") and hot != greedy
    assert hot != ids("--temperature", "5.0", "--seed", "5")
    assert ids("--repetition-penalty", "50.0") != greedy or len(set(greedy)) == len(greedy)


def test_logits_and_inspect(model_dirs, cpu_backend, capsys):
    W = P.PlainWeights(model_dirs["A"])
    ref = P.forward_logits(W, [5, 17, 3])[-1]
    assert main(["logits", "--model", str(model_dirs["A"]), "--ids", "5,17,3", *CPU]) == 0
    probe = json.loads(capsys.readouterr().out)     # src/main.rs:285-312
    assert probe["argmax"] == int(torch.argmax(ref))
    assert abs(probe["argmax_logit"] - float(ref.max())) < 1e-4
    assert len(probe["head"]) == len(probe["tail"]) == 4
    assert abs(probe["sum"] - float(ref.sum())) < 1e-3
    assert main(["inspect", "--random", "tiny-a", *CPU]) == 0
    info = json.loads(capsys.readouterr().out)
    assert (info["layers"], info["d_model"], info["vocab"], info["n_params"]) == (2, 64, 512, 141_056)


def test_a_random_model_folder_from_a_preset_and_from_a_config(tmp_path, cpu_backend, capsys):
    assert main(["random", "--out", str(tmp_path / "m"), "--preset", "tiny-b", "--seed", "5",
                 "--dtype", "float32"]) == 0
    told = json.loads(capsys.readouterr().out)
    assert (tmp_path / "m" / "config.json").exists() and (tmp_path / "m" / "model.safetensors").exists()
    assert main(["inspect", "--model", str(tmp_path / "m"), *CPU]) == 0
    assert json.loads(capsys.readouterr().out)["n_params"] == told["n_params"]
    # the same sizes from the folder's own config.json, another seed: other weights, same count
    assert main(["random", "--out", str(tmp_path / "n"), "--config", str(tmp_path / "m" / "config.json"),
                 "--seed", "6", "--bias-std", "0.02", "--dtype", "float32"]) == 0
    assert json.loads(capsys.readouterr().out)["n_params"] == told["n_params"]
    a = P.read_safetensors(tmp_path / "m" / "model.safetensors")
    b = P.read_safetensors(tmp_path / "n" / "model.safetensors")
    assert a.keys() == b.keys() and any(not torch.equal(a[k], b[k]) for k in a)
    with pytest.raises(SystemExit):
        main(["random", "--out", str(tmp_path / "x")])


def test_what_the_command_line_refuses(model_dirs, cpu_backend, capsys):
    m = str(model_dirs["A"])
    for argv, text in (
            (["generate", "--model", m, "--prompt", "hello", *CPU], "no tokenizer"),
            (["generate", "--model", m, *CPU], "--ids"),
            (["generate", "--ids", "1", *CPU], "--model DIR or --random PRESET"),
            (["generate", "--model", m, "--random", "tiny-a", "--ids", "1", *CPU], "--model DIR or --random"),
            (["generate", "--model", m, "--ids", "1", "--quant", "int8", *CPU], "not built")):
        with pytest.raises(SystemExit) as e:
            main(argv)
        assert text in str(e.value)
    # errors of the library come back as a message and exit code 1
    assert main(["generate", "--model", m, "--ids", "1,99999", *CPU]) == 1
    assert "token id outside" in capsys.readouterr().err
    assert main(["inspect", "--model", str(model_dirs["A"] / "nowhere"), *CPU]) == 1
