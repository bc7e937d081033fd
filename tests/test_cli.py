"""The command line end to end on CPU: the verbs a user types build a real engine and print a result."""
import io
import json
import os

from legion_b200.cli.main import main


def test_run_generates_from_a_random_preset(capsys):
    assert main(["run", "--model", "random:tiny-dense", "--device", "cpu", "--prompt", "hello", "-n", "5",
                 "--ignore-eos"]) == 0
    cap = capsys.readouterr()
    assert "5 generated" in cap.out + cap.err


def test_run_with_an_image_and_a_tiny_mmproj(tmp_path, capsys):
    from PIL import Image
    from legion_b200.config import PRESETS
    from legion_b200.loaders.vision import write_tiny_mmproj
    from legion_b200.vision import VisionConfig
    mm = str(tmp_path / "mmproj.gguf")
    write_tiny_mmproj(mm, VisionConfig(out_hidden=PRESETS["tiny-dense"]().hidden, patch_size=4, num_pos=16))
    img = str(tmp_path / "a.png")
    Image.new("RGB", (40, 24), (9, 200, 30)).save(img)
    assert main(["run", "--model", "random:tiny-dense", "--device", "cpu", "--mmproj", mm, "--image", img, "--prompt",
                 "what is this?", "-n", "4", "--ignore-eos"]) == 0
    cap = capsys.readouterr()
    out = cap.out + cap.err
    # 40 x 24 pixels, patches of 4 merged 2 x 2 -> 5 x 3 image tokens inside the prompt
    assert "4 generated" in out and "prompt tokens" in out
    n_prompt = int(out.split("[")[-1].split(" prompt tokens")[0])
    assert n_prompt >= 15 + len("what is this?")


def test_info_and_tokenize(capsys):
    assert main(["tokenize", "--model", "random:tiny-dense", "abc"]) == 0
    assert capsys.readouterr().out.strip()


def test_logits_dump_and_compare(tmp_path, capsys):
    """The reference-logit tool: a dump of every row, then the same prompt compared against it."""
    out = str(tmp_path / "ref.npz")
    args = ["logits", "--model", "random:tiny-hybrid-moe", "--device", "cpu", "--tokens", "5,6,7,8,9,10,11", "--all-rows"]
    assert main(args + ["--out", out]) == 0
    first = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert first["rows"] == 7 and os.path.exists(out)
    assert main(args + ["--compare", out]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    cmp = json.loads(lines[-1])
    assert cmp["max_abs_diff"] == 0.0 and cmp["argmax_agreement"] == 1.0
