"""JSON-schema constrained decoding: the automaton, the vocabulary mask and the engine integration."""
import json

import pytest
import torch

from legion_b200.grammar import Matcher, compile_response_format, compile_schema, tool_call_schema
from legion_b200.loaders.tokenizer import ByteTokenizer

SCHEMA = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"},
                                           "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "maxItems": 2},
                                           "ok": {"type": "boolean"}}, "required": ["name", "age"]}


def test_automaton_accepts_and_rejects():
    m = Matcher(compile_schema(SCHEMA), ByteTokenizer(512))
    assert m.accepts('{"name":"x","age":3}')
    assert m.accepts('{"age": -12, "name": "q\\n\\u00e9", "tags":["a","b"], "ok":true}')
    assert not m.accepts('{"name":"x"}')                      # required age missing
    assert not m.accepts('{"name":"x","age":3.5}')            # integer
    assert not m.accepts('{"name":"x","age":3,"zzz":1}')      # undeclared property
    assert not m.accepts('{"name":"x","age":3,"tags":["c"]}')
    assert not m.accepts('{"name":"x","age":3,"tags":["a","a","b"]}')
    assert not m.accepts('{"name":"x","name":"y","age":1}')   # duplicate key
    anym = Matcher(compile_schema({}), ByteTokenizer(512))
    for doc in ('{"a":[1,2.5e3,{"b":null}],"c":"d"}', '[]', '"s"', 'true', '-0.5'):
        assert anym.accepts(doc), doc
    assert not anym.accepts('{"a":}')


def test_mask_only_allows_valid_bytes():
    tok = ByteTokenizer(512)
    m = Matcher(compile_schema(SCHEMA), tok)
    allowed = m.mask().nonzero().flatten().tolist()
    assert allowed == [ord("{")]
    for ch in '{"':
        m.advance(ord(ch))
    allowed = {chr(i) for i in m.mask().nonzero().flatten().tolist()}
    assert allowed == {"n", "a", "t", "o"}                    # first letters of the declared keys
    for ch in 'age":':
        m.advance(ord(ch))
    allowed = {chr(i) for i in m.mask().nonzero().flatten().tolist()}
    assert allowed == set("-0123456789 ")
    for ch in '7,"name":"q"}':
        m.advance(ord(ch))
    assert m.finished()
    assert set(m.mask().nonzero().flatten().tolist()) == set(tok.eos_ids)


def test_tool_call_schema():
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"]}}},
        {"type": "function", "function": {"name": "noop"}}]
    m = Matcher(compile_schema(tool_call_schema(tools)), ByteTokenizer(512))
    assert m.accepts('{"name":"get_weather","arguments":{"city":"Oslo"}}')
    assert not m.accepts('{"name":"get_weather","arguments":{}}')
    assert not m.accepts('{"name":"other","arguments":{}}')
    assert m.accepts('{"name":"noop","arguments":{"x":1}}')


def test_engine_generates_valid_json_with_random_weights():
    from legion_b200.config import tiny_dense
    from legion_b200.engine.lm import EngineConfig, build_engine
    from legion_b200.engine.types import GenerateRequest, SamplingParams
    eng = build_engine(tiny_dense(), engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16))
    fmt = {"type": "json_schema", "json_schema": {"name": "p", "schema": {
        "type": "object", "properties": {"n": {"type": "integer"}, "k": {"enum": ["x", "yy"]}}, "required": ["n", "k"]}}}
    for seed in (1, 2):
        req = GenerateRequest(prompt_tokens=[1, 2, 3], response_format=fmt,
                              sampling=SamplingParams(temperature=1.0, seed=seed, max_tokens=60))
        out = eng.generate(req).collect()
        doc = json.loads(out.text)
        assert isinstance(doc["n"], int) and doc["k"] in ("x", "yy")
    with pytest.raises(ValueError):
        eng.check_response_format({"type": "json_schema", "json_schema": {"schema": {"type": "frob"}}})
    # the vocabulary masks of constrained sequences were computed by helper threads beside the forward pass
    assert getattr(eng.stats(), "masks_ahead", 0) > 10
    eng.shutdown()
