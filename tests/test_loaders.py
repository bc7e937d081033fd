"""Checkpoint formats: GGUF write/read round trip and block de-quantisation, safetensors / HF directories with
BF16, block-scaled FP8 and NVFP4 (ModelOpt and compressed-tensors layouts), tokenizer and chat template."""
import json
import os

import numpy as np
import pytest
import torch

from legion_b200.config import tiny_hybrid_moe, tiny_mla_moe, tiny_gqa_moe
from legion_b200.loaders import gguf as G
from legion_b200.loaders import quant_formats as qf
from legion_b200.loaders.gguf_map import load_gguf, write_gguf
from legion_b200.loaders.hf_map import load_hf, save_hf
from legion_b200.loaders.model import load_model
from legion_b200.loaders.safetensors_io import Checkpoint, SafetensorsFile, save_file
from legion_b200.loaders.tokenizer import BpeTokenizer, ByteTokenizer
from legion_b200.loaders import chat_template as ct
from legion_b200.models.weights import random_weights


def test_gguf_roundtrip_hybrid_model(tmp_path):
    cfg = tiny_hybrid_moe()
    w = random_weights(cfg, "cpu", torch.float32, seed=0)
    path = str(tmp_path / "m.gguf")
    write_gguf(path, cfg, w)
    cfg2, w2, md = load_gguf(path)
    assert md["general.architecture"] == "qwen35moe"
    assert cfg2.layer_kinds == cfg.layer_kinds and cfg2.n_expert == 8 and cfg2.gdn_v_heads == 4
    assert set(w2) == set(w)
    for k in w:
        assert torch.equal(w[k], w2[k]), k


def test_gguf_model_runs_same_tokens(tmp_path):
    from legion_b200.engine.lm import EngineConfig, build_engine
    cfg = tiny_hybrid_moe()
    w = random_weights(cfg, "cpu", torch.float32, seed=0, std=0.05)
    path = str(tmp_path / "m.gguf")
    write_gguf(path, cfg, w)
    cfg2, w2, tok, _ = load_model(path, "cpu")
    cfg2.gdn_tiled_heads = cfg.gdn_tiled_heads     # this file was written from ungrouped (HF-order) heads
    prompt = list(range(1, 129))
    outs = []
    for c, ww in ((cfg, w), (cfg2, w2)):
        e = build_engine(c, weights=ww, engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16))
        outs.append(e.generate_text(tokens=prompt, max_tokens=8, ignore_eos=True).token_ids)
        e.shutdown()
    assert outs[0] == outs[1]


def _ref_dequant(name, blk):
    """Scalar re-statement of the block formats (independent of the vectorised code)."""
    f16 = lambda b: float(np.frombuffer(bytes(b), dtype=np.float16)[0])
    out = []
    if name == "Q8_0":
        d = f16(blk[0:2])
        return [d * int(np.int8(x)) for x in blk[2:34]]
    if name == "Q4_0":
        d = f16(blk[0:2])
        q = blk[2:18]
        return [d * ((int(x) & 15) - 8) for x in q] + [d * ((int(x) >> 4) - 8) for x in q]
    def sm(j, s):
        if j < 4:
            return s[j] & 63, s[j + 4] & 63
        return (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4), (s[j + 4] >> 4) | ((s[j] >> 6) << 4)
    if name == "Q4_K":
        d, dmin, s, q = f16(blk[0:2]), f16(blk[2:4]), [int(x) for x in blk[4:16]], [int(x) for x in blk[16:144]]
        for i in range(4):
            sc1, m1 = sm(2 * i, s)
            sc2, m2 = sm(2 * i + 1, s)
            ch = q[32 * i:32 * i + 32]
            out += [d * sc1 * (x & 15) - dmin * m1 for x in ch] + [d * sc2 * (x >> 4) - dmin * m2 for x in ch]
        return out
    if name == "Q5_K":
        d, dmin, s = f16(blk[0:2]), f16(blk[2:4]), [int(x) for x in blk[4:16]]
        qh, q = [int(x) for x in blk[16:48]], [int(x) for x in blk[48:176]]
        for i in range(4):
            sc1, m1 = sm(2 * i, s)
            sc2, m2 = sm(2 * i + 1, s)
            ch = q[32 * i:32 * i + 32]
            out += [d * sc1 * ((x & 15) + (16 if qh[l] & (1 << (2 * i)) else 0)) - dmin * m1 for l, x in enumerate(ch)]
            out += [d * sc2 * ((x >> 4) + (16 if qh[l] & (2 << (2 * i)) else 0)) - dmin * m2 for l, x in enumerate(ch)]
        return out
    if name == "Q6_K":
        ql, qh = [int(x) for x in blk[0:128]], [int(x) for x in blk[128:192]]
        sc = [int(np.int8(x)) for x in blk[192:208]]
        d = f16(blk[208:210])
        y = [0.0] * 256
        for n in range(2):
            for l in range(32):
                i = l // 16
                a, b, c, e = ql[64 * n + l], ql[64 * n + l + 32], qh[32 * n + l], sc[8 * n:8 * n + 8]
                y[128 * n + l] = d * e[i] * (((a & 15) | ((c & 3) << 4)) - 32)
                y[128 * n + l + 32] = d * e[i + 2] * (((b & 15) | (((c >> 2) & 3) << 4)) - 32)
                y[128 * n + l + 64] = d * e[i + 4] * (((a >> 4) | (((c >> 4) & 3) << 4)) - 32)
                y[128 * n + l + 96] = d * e[i + 6] * (((b >> 4) | (((c >> 6) & 3) << 4)) - 32)
        return y
    raise AssertionError(name)


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0", "Q4_K", "Q5_K", "Q6_K"])
def test_gguf_dequant_matches_scalar_reference(name):
    rng = np.random.default_rng(3)
    tid = G.TYPE_ID[name]
    _, be, bb = G.GGML_TYPES[tid]
    raw = rng.integers(0, 256, size=(6, bb), dtype=np.uint8)
    # keep the f16 scale fields finite
    for off in ([0] if name in ("Q8_0", "Q4_0") else ([0, 2] if name in ("Q4_K", "Q5_K") else [208])):
        raw[:, off:off + 2] = np.frombuffer(np.float16(rng.uniform(-2, 2, 6)).tobytes(), dtype=np.uint8).reshape(6, 2)
    got = G.dequantize(raw.reshape(-1), tid, (6, be))
    want = np.array([_ref_dequant(name, row) for row in raw], dtype=np.float32)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    try:
        from gguf import quants as gq
        lib = gq.dequantize(raw, tid)
        np.testing.assert_allclose(got, lib.reshape(6, be), rtol=1e-5, atol=1e-5)
    except Exception:
        pass


def test_gguf_quantised_write_read(tmp_path):
    x = np.random.default_rng(0).standard_normal((8, 64)).astype(np.float32)
    wr = G.GgufWriter(str(tmp_path / "q.gguf"), "test")
    wr.add("test.ints", [1, 2, 3])
    wr.add("test.name", "héllo")
    wr.add_tensor("a", x, "Q8_0")
    wr.add_tensor("b", x, "Q4_0")
    wr.add_tensor("c", torch.from_numpy(x).bfloat16())
    wr.add_tensor("d", x, "F16")
    wr.write()
    g = G.GgufFile(str(tmp_path / "q.gguf"))
    assert g.metadata["test.ints"] == [1, 2, 3] and g.metadata["test.name"] == "héllo"
    assert g.tensors["a"].type_name == "Q8_0" and g.tensors["a"].shape == (8, 64)
    assert np.abs(g.numpy("a") - x).max() < 0.03
    assert np.abs(g.numpy("b") - x).max() < 0.5
    assert np.abs(g.numpy("c") - x).max() < 0.02 and np.abs(g.numpy("d") - x).max() < 2e-3


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(4, 4).bfloat16(), "c": torch.arange(6, dtype=torch.int32),
         "d": torch.randn(8, 16).to(torch.float8_e4m3fn), "e": torch.randint(0, 255, (2, 8), dtype=torch.uint8)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p, {"format": "pt"})
    f = SafetensorsFile(p)
    assert f.metadata == {"format": "pt"}
    for k, v in t.items():
        got = f.tensor(k)
        assert got.dtype == v.dtype and torch.equal(got.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else got,
                                                    v.view(torch.uint8) if v.dtype == torch.float8_e4m3fn else v)
    from safetensors.torch import load_file      # the reference implementation reads our file
    lib = load_file(p)
    assert torch.equal(lib["a"], t["a"]) and torch.equal(lib["b"], t["b"])


def test_nvfp4_and_fp8_golden_vectors():
    # codes 0..15 with scale 1 decode to the E2M1 table
    codes = torch.tensor([[0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]], dtype=torch.uint8)
    one = torch.tensor([[1.0]]).to(torch.float8_e4m3fn)
    out = qf.nvfp4_dequant(codes, one, 2.0)
    assert out.tolist() == [[0, 1, 2, 3, 4, 6, 8, 12, -0.0, -1, -2, -3, -4, -6, -8, -12]]
    out_ct = qf.nvfp4_dequant(codes, one, 0.5, global_is_divisor=True)
    assert torch.equal(out, out_ct)
    w = torch.randn(32, 64) * 0.02
    c, s, g = qf.nvfp4_quant(w)
    back = qf.nvfp4_dequant(c, s, g)
    assert (back - w).norm() / w.norm() < 0.12
    q, sc = qf.fp8_block_quant(torch.randn(200, 300))
    assert q.shape == (200, 300) and sc.shape == (2, 3)
    w8 = torch.randn(200, 300)
    q, sc = qf.fp8_block_quant(w8)
    assert (qf.fp8_dequant(q, sc, (128, 128)) - w8).norm() / w8.norm() < 0.04
    xq, xs = qf.fp8_act_quant(torch.randn(5, 256))
    assert xs.shape == (5, 2)


@pytest.mark.parametrize("quant,tol", [("none", 0.01), ("fp8_block", 0.05), ("nvfp4", 0.15), ("nvfp4_ct", 0.15)])
@pytest.mark.parametrize("mk", [tiny_hybrid_moe, tiny_mla_moe, tiny_gqa_moe])
def test_hf_directory_roundtrip(tmp_path, mk, quant, tol):
    cfg = mk()
    cfg.mtp_layers = 0
    w = random_weights(cfg, "cpu", torch.float32, seed=1)
    d = str(tmp_path / "ck")
    save_hf(d, cfg, w, quant=quant, dtype=torch.float32 if quant == "none" else torch.bfloat16)
    ck = Checkpoint(d)
    assert ck.quant_method() == {"none": "none", "fp8_block": "fp8_block", "nvfp4": "nvfp4", "nvfp4_ct": "nvfp4_ct"}[quant]
    cfg2, w2, _ = load_hf(d)
    assert cfg2.layer_kinds == cfg.layer_kinds and cfg2.n_expert == cfg.n_expert and cfg2.kv_lora == cfg.kv_lora
    assert set(w2) == set(w)
    for k in w:
        a, b = w[k].float(), w2[k].float()
        assert a.shape == b.shape, k
        if a.dim() >= 2 and quant != "none":
            assert (a - b).norm() <= tol * a.norm() + 1e-6, k
        else:
            assert torch.allclose(a, b, atol=2e-3, rtol=1e-2), k


def test_byte_tokenizer_and_bpe():
    t = ByteTokenizer(512)
    ids = t.encode("hi<|im_end|>é")
    assert ids[:2] == [104, 105] and ids[2] == 259 and t.decode(ids) == "hi<|im_end|>é"
    assert t.decode(ids, skip_special=True) == "hié"
    # a small BPE: bytes + merges "h e" "he l" "l o"
    from legion_b200.loaders.tokenizer import _byte_to_unicode
    b2u = _byte_to_unicode()
    tokens = [b2u[i] for i in range(256)] + ["he", "hel", "lo", "Ġw", "<|eot|>"]
    bpe = BpeTokenizer(tokens, ["h e", "he l", "l o", "Ġ w"], token_types=[1] * 260 + [3], eos_ids=[260])
    ids = bpe.encode("hello world<|eot|>")
    assert [bpe.tokens[i] for i in ids[:2]] == ["hel", "lo"] and ids[-1] == 260
    assert bpe.decode(ids) == "hello world<|eot|>" and bpe.decode(ids, skip_special=True) == "hello world"
    assert bpe.token_bytes(ids[0]) == b"hel"
    md = {"tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": ["h e"], "tokenizer.ggml.eos_token_id": 260,
          "tokenizer.ggml.token_type": [1] * 260 + [3]}
    assert BpeTokenizer.from_gguf_metadata(md).eos_ids == (260,)


def test_chat_template_rendering():
    from legion_b200.loaders.tokenizer import DEFAULT_CHATML_TEMPLATE
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
    out = ct.render(DEFAULT_CHATML_TEMPLATE, msgs)
    assert out == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    no_think = ct.render(DEFAULT_CHATML_TEMPLATE, msgs, enable_thinking=False)
    assert no_think.endswith("<think>\n\n</think>\n\n")
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object"}}}]
    with_tools = ct.render(DEFAULT_CHATML_TEMPLATE, msgs + [
        {"role": "assistant", "content": "", "tool_calls": [{"id": "1", "function": {"name": "f", "arguments": "{\"a\": 1}"}}]},
        {"role": "tool", "content": "42"}], tools=tools)
    assert "<tools>" in with_tools and '"name": "f", "arguments": {"a": 1}' in with_tools and "<tool_response>\n42" in with_tools
    with pytest.raises(ct.TemplateError):
        ct.render("{{ raise_exception('nope') }}", msgs)


def test_native_bpe_merges_equal_python():
    """The C++ merge loop of the host runtime and the Python one give the same ids (unknown pieces included)."""
    import random
    from legion_b200.loaders.tokenizer import BpeTokenizer, _byte_to_unicode
    b2u = _byte_to_unicode()
    rng = random.Random(0)
    toks = [b2u[i] for i in range(256) if i != ord("z")]          # 'z' is unknown: falls out of the ids
    merges = []
    for _ in range(2000):
        a, b = rng.choice(toks), rng.choice(toks)
        if a + b not in toks and len(a + b) < 10:
            toks.append(a + b)
            merges.append(a + " " + b)
    t = BpeTokenizer(toks, merges)
    if t._native is None:
        pytest.skip("native host runtime not built")
    text = "".join(rng.choice("abcdefghij klmnop\nqrstuvz 0123 éü漢字") for _ in range(5000))
    got = t.encode(text)
    t._native = None
    t._cache.clear()
    assert got == t.encode(text) and len(got) > 1000


def test_hf_directory_expert_range_reads_only_those_experts(tmp_path):
    """An expert-parallel rank opens the same directory with its expert range and gets exactly that slice."""
    cfg = tiny_gqa_moe()
    w = random_weights(cfg, "cpu", torch.float32, seed=4)
    d = str(tmp_path / "ck")
    save_hf(d, cfg, w, quant="none", dtype=torch.float32)
    _, full, _ = load_hf(d)
    lo, hi = 2, 6
    _, part, _ = load_hf(d, expert_range=(lo, hi))
    for k, v in full.items():
        if k.endswith(("moe.gate_up", "moe.down")):
            assert part[k].shape[0] == hi - lo and torch.equal(part[k], v[lo:hi])
        else:
            assert torch.equal(part[k], v)


def test_parallel_read_ahead_gives_the_same_tensors(tmp_path):
    """Layer tensors read ahead by a pool of positional reads (several pieces per tensor) equal the memory-mapped
    ones; with an expert range only those experts are read."""
    cfg = tiny_gqa_moe()
    w = random_weights(cfg, "cpu", torch.float32, seed=6)
    d = str(tmp_path / "ck")
    save_hf(d, cfg, w, quant="none", dtype=torch.float32)
    _, plain, _ = load_hf(d)
    _, ahead, _ = load_hf(d, read_threads=4)
    assert set(plain) == set(ahead) and all(torch.equal(plain[k], ahead[k]) for k in plain)
    ck = Checkpoint(d)
    name = next(n for n in ck.names() if n.endswith("experts.3.down_proj.weight"))
    n = ck.prefetch([name], threads=3, chunk=1000)          # many small pieces of one tensor
    assert n == ck.get(name).numel() * 4 or n > 0
    ck2 = Checkpoint(d)
    assert torch.equal(Checkpoint(d).get(name), (ck2.prefetch([name], threads=2, chunk=777), ck2.get(name))[1])
    _, part, ck3 = load_hf(d, expert_range=(2, 4), read_threads=2)
    assert part["l0.moe.gate_up"].shape[0] == 2 and torch.equal(part["l0.moe.gate_up"], plain["l0.moe.gate_up"][2:4])
    assert not ck3._ahead or all(".experts." not in k or k.split(".experts.")[1].split(".")[0] in ("2", "3") for k in ck3._ahead)


def test_hardware_keyed_engine_defaults():
    """Sizes the command line leaves open follow what the device reports."""
    from legion_b200.hw.defaults import engine_defaults
    cpu = engine_defaults("cpu")
    assert (cpu.profile, cpu.kv_block, cpu.prefill_chunk, cpu.cuda_graphs) == ("cpu", 16, 512, False)
    b200 = engine_defaults("cuda:0", total_gib=179.0)
    assert (b200.profile, b200.prefill_chunk, b200.kv_block, b200.max_batch_tokens) == ("b200", 8192, 64, 8192)
    assert engine_defaults("cuda", total_gib=79.0).prefill_chunk == 4096
    small = engine_defaults("cuda", total_gib=23.0)
    assert small.profile == "small" and small.max_seqs < b200.max_seqs and small.gpu_memory_utilization < 0.9


def test_sentencepiece_style_tokenizer_from_gguf_metadata():
    """Score-ordered merges, U+2581 spaces, byte fallback, control pieces; against the `sentencepiece` package on a
    model trained here when it is importable, else against hand-checked merges."""
    from legion_b200.loaders.tokenizer import SpmTokenizer, tokenizer_from_gguf_metadata
    sp = "\u2581"
    pieces = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + [
        sp, "h", "e", "l", "o", "w", "r", "d", sp + "h", "he", "ll", sp + "he", "llo", sp + "hello", sp + "w", "or", "ld",
        sp + "wor", sp + "world", "<start_of_turn>"]
    scores = [0.0] * 259 + [-1.0, -2, -2, -2, -2, -2, -2, -2, -1.5, -1.2, -1.1, -0.9, -0.8, -0.5, -1.4, -1.3, -1.25, -0.7, -0.4,
                            0.0]
    types = [2, 3, 3] + [6] * 256 + [1] * 19 + [4]
    md = {"tokenizer.ggml.model": "llama", "tokenizer.ggml.tokens": pieces, "tokenizer.ggml.scores": scores,
          "tokenizer.ggml.token_type": types, "tokenizer.ggml.bos_token_id": 1, "tokenizer.ggml.eos_token_id": 2,
          "tokenizer.ggml.add_bos_token": True}
    tok = tokenizer_from_gguf_metadata(md)
    assert isinstance(tok, SpmTokenizer)
    ids = tok.encode("hello world", add_special=True)
    assert ids == [1, pieces.index(sp + "hello"), pieces.index(sp + "world")]
    assert tok.decode(ids, skip_special=True) == "hello world"
    # a character no piece covers falls back to its UTF-8 bytes; control pieces are matched as text
    ids = tok.encode("<start_of_turn>h\u00e9", add_special=False)
    assert ids[0] == pieces.index("<start_of_turn>")
    assert [pieces[i] for i in ids[1:]] == [sp + "h", "<0xC3>", "<0xA9>"] or [pieces[i] for i in ids[1:]] == [sp, "h", "<0xC3>", "<0xA9>"]
    assert tok.decode(ids[1:]) == "h\u00e9"
    assert tok.token_to_id("<start_of_turn>") == pieces.index("<start_of_turn>")
    try:
        import sentencepiece as spm
    except ImportError:
        return
    import io
    text = ("the quick brown fox jumps over the lazy dog. " * 40 + "pack my box with five dozen liquor jugs. " * 40)
    model = io.BytesIO()
    spm.SentencePieceTrainer.train(sentence_iterator=iter(text.split(". ")), model_writer=model, vocab_size=340,
                                   model_type="bpe", byte_fallback=True, character_coverage=1.0, bos_id=1, eos_id=2,
                                   unk_id=0, minloglevel=2, normalization_rule_name="identity",
                                   remove_extra_whitespaces=False)
    ref = spm.SentencePieceProcessor(model_proto=model.getvalue())
    n = ref.get_piece_size()
    toks = [ref.id_to_piece(i) for i in range(n)]
    sc = [ref.get_score(i) for i in range(n)]
    ty = [2 if ref.is_unknown(i) else 3 if ref.is_control(i) else 6 if ref.is_byte(i) else 1 for i in range(n)]
    mine = SpmTokenizer(toks, sc, ty, bos_id=1, eos_ids=(2,), add_bos=False)
    for s in ("the lazy dog jumps", "five quick boxes", "liquor\u00e9 jugs!", "  two  spaces"):
        assert mine.encode(s) == ref.encode(s), s
        assert mine.decode(mine.encode(s)) == ref.decode(ref.encode(s)), s


def test_long_prompts_encode_their_pretokens_in_parallel():
    """Texts past ``PARALLEL_CHARS`` cut their pre-tokens once and encode contiguous runs of them on several threads
    in the native runtime: same ids as the serial loop, special tokens in between included."""
    import collections
    import random
    from legion_b200.loaders.tokenizer import BpeTokenizer, _byte_to_unicode
    b2u = _byte_to_unicode()
    words = ["the", "quick", "brown", "fox", "jumps", "over", "lazy", "dog", "tokenizer", "h\u00e9llo", "\u00dcn\u00efcode"]
    corp = [[b2u[b] for b in (" " + w).encode()] for w in words]
    toks, merges = [b2u[b] for b in range(256)], []
    for _ in range(100):
        cnt = collections.Counter((a, b) for w in corp for a, b in zip(w, w[1:]))
        if not cnt:
            break
        (a, b), _n = cnt.most_common(1)[0]
        merges.append(a + " " + b)
        toks.append(a + b)
        for w in corp:
            i = 0
            while i + 1 < len(w):
                if w[i] == a and w[i + 1] == b:
                    w[i:i + 2] = [a + b]
                else:
                    i += 1
    toks.append("<|sep|>")
    tok = BpeTokenizer(toks, merges, pre="gpt2", extra_special=["<|sep|>"])
    if tok._native is None or not hasattr(tok._native, "encode_pieces"):
        import pytest
        pytest.skip("native host runtime not built")
    rng = random.Random(0)
    text = " ".join(rng.choice(words) + rng.choice(["", ",", ".", "\n", "  ", "123", "<|sep|>"]) for _ in range(9000))
    assert len(text) > tok.PARALLEL_CHARS
    par = tok.encode(text)
    tok.PARALLEL_CHARS = 1 << 60
    tok._cache.clear()
    assert tok.encode(text) == par
    assert tok.decode(par) == text


def test_vision_language_config_carries_the_rotary_sections():
    from legion_b200.loaders.hf_map import config_from_hf
    c = config_from_hf({"model_type": "qwen3_5_moe", "text_config": {
        "model_type": "qwen3_5_moe_text", "num_attention_heads": 4, "hidden_size": 256, "num_hidden_layers": 4,
        "vocab_size": 1000, "num_key_value_heads": 2, "head_dim": 64, "partial_rotary_factor": 1.0,
        "rope_parameters": {"rope_type": "default", "rope_theta": 5e6, "mrope_section": [11, 11, 10], "mrope_interleaved": True},
        "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 64, "shared_expert_intermediate_size": 64},
        "vision_config": {"depth": 2}})
    assert c.mrope_sections == (11, 11, 10) and c.mrope_interleaved and c.rope_theta == 5e6 and c.arch == "qwen35moe"


def test_gemma4_tokenizer_against_the_tokenizers_library(tmp_path):
    """Raw-text BPE with byte fallback (Gemma 4's kind): a small vocabulary trained with the ``tokenizers`` library
    (spaces as U+2581, cut at newline runs, ``<0xXX>`` byte tokens) saved as ``tokenizer.json``, loaded by
    ``BpeTokenizer.from_hf_dir`` (which picks ``Gemma4Tokenizer`` for it): same ids as the library on text with unseen
    characters, newline runs and markers; markers that are not control tokens stay in decoded text."""
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Regex, decoders, models, normalizers, pre_tokenizers, trainers
    from legion_b200.loaders.tokenizer import BpeTokenizer, Gemma4Tokenizer
    t = tk.Tokenizer(models.BPE(byte_fallback=True, unk_token="<unk>", fuse_unk=False))
    t.normalizer = normalizers.Replace(" ", "▁")
    t.pre_tokenizer = pre_tokenizers.Split(Regex("[^\\n]+|\\n+"), behavior="isolated")
    t.decoder = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse()])
    specials = ["<pad>", "<eos>", "<bos>", "<unk>"] + [f"<0x{b:02X}>" for b in range(256)]
    corpus = ["the quick brown fox jumps over the lazy dog\n\nand then it  sleeps\n", "hello world, hello there\n",
              "def f(x):\n    return x + 1\n\n\nprint(f(2))\n", "a b c d e f g the then there"] * 4
    t.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=420, special_tokens=specials, show_progress=False))
    t.add_special_tokens(["<turn|>"])
    t.add_tokens(["<|channel>", "<channel|>", "<|tool_call>"])
    t.save(str(tmp_path / "tokenizer.json"))
    json.dump({"bos_token": "<bos>", "eos_token": "<eos>"}, open(tmp_path / "tokenizer_config.json", "w"))
    mine = BpeTokenizer.from_hf_dir(str(tmp_path))
    assert isinstance(mine, Gemma4Tokenizer) and mine.add_bos
    for text in ("the lazy dog sleeps", "hello  there\n\nworld", "café \U0001F600 ok", "\n\n\nx = f(2)\n",
                 "<|channel>thought\nhm<channel|>hello<turn|>", "  leading and trailing  "):
        want = t.encode(text, add_special_tokens=False).ids
        assert mine.encode(text) == want, text
        assert mine.decode(want) == t.decode(want, skip_special_tokens=False), text
    ids = mine.encode("<|channel>thought\nhm<channel|>ok<turn|>")
    assert mine.decode(ids, skip_special=True) == "<|channel>thought\nhm<channel|>ok"
    assert mine.encode("x", add_special=True)[0] == mine.vocab["<bos>"]
    assert mine.vocab["<turn|>"] in mine.eos_ids


def test_chat_format_is_read_from_the_vocabulary():
    from legion_b200.engine.text import ChatFormat

    class Tok:
        def __init__(self, names):
            self.ids = {n: i for i, n in enumerate(names)}

        def token_to_id(self, t):
            return self.ids.get(t)

    g = ChatFormat(Tok(["<|channel>", "<channel|>", "<|tool_call>", "<turn|>", "<|tool_response>"]))
    assert (g.kind, g.tool_format, g.tags) == ("gemma4", "gemma4", ("<|channel>thought", "<channel|>"))
    assert g.stop_ids == (3, 4)
    assert g.starts_in_reasoning("<|turn>model\n<|channel>thought\n") and not g.starts_in_reasoning("<|turn>model\n")
    assert not g.starts_in_reasoning("<|turn>model\n<|channel>thought\n<channel|>")
    sp = g.splitter("")
    assert sp.push("<|channel>thought\nplan<channel|>answer") == [("reasoning", "\nplan"), ("text", "answer")]
    glm = ChatFormat(Tok(["<tool_call>", "<arg_key>", "<arg_value>", "<think>", "<|observation|>"]))
    assert (glm.kind, glm.tool_format, glm.stop_ids) == ("glm", "glm", (4,))
    assert glm.starts_in_reasoning("<|assistant|>\n<think>") and not glm.starts_in_reasoning("<think>a</think>\nb")
    q = ChatFormat(Tok(["<|im_end|>", "<think>"]), tool_format="hermes")
    assert (q.kind, q.tool_format, q.stop_ids) == ("plain", "hermes", (0,))
    assert q.starts_in_reasoning("<|im_start|>assistant\n<think>\n")
    assert not ChatFormat(Tok(["a"])).starts_in_reasoning("<think>")


@pytest.mark.parametrize("pre", ["qwen2", "llama3", "gpt2"])
def test_byte_level_bpe_against_the_tokenizers_library(tmp_path, pre):
    """Byte-level BPE: a vocabulary trained with the ``tokenizers`` library behind the family's pre-tokeniser pattern,
    saved as ``tokenizer.json`` and loaded here, gives that library's ids on contractions, digit runs, whitespace
    runs, newlines, punctuation and non-Latin text; the long-text path (pre-tokens encoded on several threads) gives
    the same ids as the serial loop."""
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Regex, decoders, models, pre_tokenizers, trainers
    from legion_b200.loaders.tokenizer import PRE_PATTERNS, BpeTokenizer
    t = tk.Tokenizer(models.BPE())
    t.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(PRE_PATTERNS[pre]), behavior="isolated", invert=False),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    t.decoder = decoders.ByteLevel()
    corpus = ["The quick brown fox doesn't jump over 12345 lazy dogs!  It's 3.14159...\n\n\tIndented line\r\n",
              "def f(x):\n    return x + 1  # comment\n\n\nprint(f(2))\n", "naïve café — “quotes” and emoji \U0001F600 ok",
              "Привет, мир! 你好，世界。 こんにちは", "a  b   c    d\n \n  \n", "I'LL we'Ve THEY'RE x's"] * 3
    t.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=600, show_progress=False,
                                                      initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                                      special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"]))
    t.save(str(tmp_path / "tokenizer.json"))
    mine = BpeTokenizer.from_hf_dir(str(tmp_path))
    assert mine.pat.pattern == PRE_PATTERNS[pre]              # read from the file's pre-tokeniser
    texts = corpus[:6] + ["  leading", "trailing  ", "x\n\n\ny", "1234567 89", "<|im_start|>user\nhi<|im_end|>\n",
                          "tabs\t\tand spaces  \n", "can't won't I'd they'll", "end.\n"]
    for text in texts:
        want = t.encode(text, add_special_tokens=False).ids
        assert mine.encode(text) == want, (pre, text)
        assert mine.decode(want) == t.decode(want, skip_special_tokens=False)
    long = " ".join(corpus) * 50
    assert len(long) >= mine.PARALLEL_CHARS
    assert mine.encode(long) == t.encode(long, add_special_tokens=False).ids


@pytest.mark.parametrize("preset", ["tiny-hybrid-moe", "tiny-mla-moe"])
def test_hf_checkpoints_carry_the_draft_head(tmp_path, preset):
    """The MTP head in Hugging Face naming (``mtp.*`` for the hybrid family, layer ``n_layer`` with ``eh_proj`` /
    ``enorm`` / ``hnorm`` / ``shared_head.norm`` for DeepSeek): written, read back tensor for tensor, and drafting
    with it equals plain greedy decoding; a checkpoint without the head loads with the flag cleared."""
    from legion_b200.config import PRESETS
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.loaders.hf_map import load_hf, save_hf
    from legion_b200.models.weights import random_weights
    cfg = PRESETS[preset]()
    cfg.mtp_layers = 1
    w = random_weights(cfg, "cpu", torch.float32, seed=2, std=0.05)
    assert "mtp0.eh_proj" in w
    d1 = str(tmp_path / "with")
    save_hf(d1, cfg, w, dtype=torch.float32)
    cfg2, w2, _ = load_hf(d1, "cpu", torch.float32)
    assert cfg2.mtp_layers == 1 and set(w2) == set(w)
    for k in w:
        assert torch.allclose(w[k].float(), w2[k].float(), atol=1e-6), k
    ec = dict(ctx_size=256, max_seqs=2, block_size=16, max_batch_tokens=128)
    toks = list(range(7, 60))
    plain = build_engine(cfg2, weights=dict(w2), engine_cfg=EngineConfig(**ec))
    want = plain.generate_text(tokens=toks, max_tokens=12, ignore_eos=True).token_ids
    plain.shutdown()
    spec = build_engine(cfg2, weights=dict(w2), engine_cfg=EngineConfig(spec="mtp", spec_k=2, **ec))
    got = spec.generate_text(tokens=toks, max_tokens=12, ignore_eos=True).token_ids
    spec.shutdown()
    assert got == want
    d2 = str(tmp_path / "without")
    save_hf(d2, cfg, {k: v for k, v in w.items() if not k.startswith("mtp")}, dtype=torch.float32)
    cfg3, w3, _ = load_hf(d2, "cpu", torch.float32)
    assert cfg3.mtp_layers == 0 and not any(k.startswith("mtp") for k in w3)


def test_gguf_codecs_and_files_against_the_gguf_package(tmp_path):
    """llama.cpp's own Python package as the oracle: block formats it can encode (Q8_0, Q4_0, Q4_1, Q5_0, Q5_1) and
    random well-formed blocks of those it can only decode (Q2_K .. Q6_K, IQ4_NL) expand to the same floats bit for
    bit; a file it writes (metadata of every kind, F32 / F16 / Q8_0 tensors) reads back here, and a file written
    here reads back there."""
    gguf = pytest.importorskip("gguf")
    from gguf import GGMLQuantizationType as T, quants
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((8, 512)) * 0.7).astype(np.float32)
    for name in ("Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1"):
        raw = quants.quantize(x, getattr(T, name))
        got = G.dequantize(np.frombuffer(raw.tobytes(), dtype=np.uint8), G.TYPE_ID[name], x.shape)
        assert np.array_equal(got, quants.dequantize(raw, getattr(T, name))), name
    f16_at = {"Q4_K": (0, 2), "Q5_K": (0, 2), "Q6_K": (208,), "Q2_K": (80, 82), "Q3_K": (108,), "IQ4_NL": (0,)}
    for name, offs in f16_at.items():
        tid = G.TYPE_ID[name]
        _, be, bb = G.GGML_TYPES[tid]
        raw = rng.integers(0, 256, size=(24, bb), dtype=np.uint8)
        for off in offs:
            raw[:, off:off + 2] = (rng.standard_normal(24) * 0.1).astype(np.float16).view(np.uint8).reshape(24, 2)
        want = quants.dequantize(raw.reshape(4, -1), getattr(T, name))
        got = G.dequantize(raw.reshape(-1), tid, (4, 24 * be // 4))
        assert np.array_equal(got, want), name
    p = str(tmp_path / "theirs.gguf")
    wr = gguf.GGUFWriter(p, "llama")
    wr.add_uint32("llama.block_count", 2)
    wr.add_string("general.name", "x")
    wr.add_array("tokenizer.ggml.tokens", ["a", "b", "c"])
    wr.add_float32("llama.rope.freq_base", 10000.0)
    wr.add_bool("flag", True)
    wr.add_tensor("a.weight", x)
    wr.add_tensor("b.weight", quants.quantize(x, T.Q8_0), raw_dtype=T.Q8_0)
    wr.add_tensor("c.weight", x.astype(np.float16))
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    f = G.GgufFile(p)
    md = f.metadata
    assert (md["llama.block_count"], md["general.name"], md["tokenizer.ggml.tokens"], md["flag"]) == (2, "x", ["a", "b", "c"], True)
    assert abs(md["llama.rope.freq_base"] - 10000.0) < 1e-3
    assert np.array_equal(f.torch("a.weight").numpy(), x)
    assert np.array_equal(f.torch("b.weight").numpy(), quants.dequantize(quants.quantize(x, T.Q8_0), T.Q8_0))
    assert np.array_equal(f.torch("c.weight").numpy(), x.astype(np.float16).astype(np.float32))
    p2 = str(tmp_path / "mine.gguf")
    w2 = G.GgufWriter(p2, "llama")
    w2.add("llama.block_count", 3)
    w2.add("general.name", "mine")
    w2.add("arr", [1, 2, 3])
    w2.add("names", ["x", "yy"])
    w2.add_tensor("t.weight", torch.from_numpy(x))
    w2.add_tensor("q.weight", torch.from_numpy(x), "Q8_0")
    w2.write()
    r = gguf.GGUFReader(p2)
    fields = {k: v.contents() for k, v in r.fields.items() if not k.startswith("GGUF")}
    assert fields["llama.block_count"] == 3 and fields["general.name"] == "mine"
    assert fields["arr"] == [1, 2, 3] and fields["names"] == ["x", "yy"]
    by_name = {t.name: t for t in r.tensors}
    assert np.array_equal(np.asarray(by_name["t.weight"].data).reshape(x.shape), x)
    q = by_name["q.weight"]
    assert q.tensor_type == T.Q8_0
    assert np.array_equal(quants.dequantize(q.data, q.tensor_type).reshape(x.shape),
                          quants.dequantize(quants.quantize(x, T.Q8_0), T.Q8_0))


@pytest.mark.parametrize("preset", ["tiny-hybrid-moe", "tiny-gqa-moe", "tiny-dense", "tiny-mla-moe", "tiny-gemma4"])
def test_gguf_tensor_names_are_the_ones_llama_cpp_lists(preset):
    """Every tensor name the GGUF writer emits for an architecture is in the ``gguf`` package's table for it (the
    draft head's ``nextn.*`` tensors of a latent-attention model excepted: llama.cpp lists them for other families
    only)."""
    import re
    gguf = pytest.importorskip("gguf")
    from legion_b200.config import PRESETS
    from legion_b200.loaders.gguf_map import ARCH_TO_GGUF, to_gguf_tensors
    from legion_b200.models.weights import random_weights
    cfg = PRESETS[preset]()
    names = to_gguf_tensors(cfg, random_weights(cfg, "cpu", torch.float32, seed=0))
    arch = {v: k for k, v in gguf.MODEL_ARCH_NAMES.items()}[ARCH_TO_GGUF[cfg.arch]]
    allowed = {gguf.TENSOR_NAMES[t] for t in gguf.MODEL_TENSORS[arch]}
    for n in names:
        base = re.sub(r"\.(weight|bias|scale)$", "", re.sub(r"^blk\.\d+\.", "blk.{bid}.", n))
        assert base in allowed or ".nextn." in base, n
