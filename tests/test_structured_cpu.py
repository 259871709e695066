"""Decoding constrained to a JSON schema: the incremental matcher and its use by the engine."""

import json

import pytest
import torch

from parallax_b200.engine.structured import JsonSchemaMatcher, TokenChooser

PERSON = {"type": "object",
          "properties": {"name": {"type": "string", "minLength": 1},
                         "age": {"type": "integer"},
                         "tags": {"type": "array", "items": {"type": "string"}, "maxItems": 2},
                         "kind": {"enum": ["cat", "dog", 7]},
                         "score": {"type": ["number", "null"]}},
          "required": ["name", "age"]}


def _full(schema, text):
    m = JsonSchemaMatcher(schema)
    return m.advance(text) and m.done


@pytest.mark.parametrize("text", [
    '{"name":"Bo","age":3}',
    '{ "name" : "B\\u00e9 \\"x\\"", "age": -12 , "tags": ["a","b"], "kind": "dog", "score": 1.5e-3 }',
    '{"name":"x","age":0,"kind":7,"score":null}',
    '{"name":"x","age":10,"tags":[]}\n',
])
def test_valid_documents_are_accepted(text):
    assert _full(PERSON, text)
    json.loads(text)


@pytest.mark.parametrize("text", [
    '{"age":3}',                       # required name missing: '}' refused
    '{"name":"","age":3}',            # minLength
    '{"name":"x","age":3.5}',          # integer
    '{"name":"x","age":3,"tags":["a","b","c"]}',     # maxItems
    '{"name":"x","age":3,"kind":"bird"}',            # enum
    '{"name":"x","age":3,"extra":1}',                # undeclared key
    '{"age":3,"name":"x"}',                          # keys come in the order of the schema
    '{"name":"x","age":03}',                         # leading zero
    '["name"]',
])
def test_invalid_documents_are_refused_at_the_offending_character(text):
    m = JsonSchemaMatcher(PERSON)
    ok = m.advance(text)
    assert not (ok and m.done)


def test_prefixes_and_completion():
    m = JsonSchemaMatcher(PERSON)
    doc = '{"name":"Al","age":41,"score":2}'
    for i, ch in enumerate(doc):
        assert not m.done
        assert m.accepts(ch), (i, ch)
        assert m.advance(ch)
    assert m.done and m.accepts(" ") and not m.accepts("x")
    # a number at the top level ends at whitespace or at the end of the text
    n = JsonSchemaMatcher({"type": "number"})
    assert n.advance("12") and not n.done and n.can_finish_with(" ") and n.advance(".5 ") and n.done


def test_any_value_refs_recursion_and_alternatives():
    assert _full(True, '{"a":[1,{"b":null}],"c":"d"}')
    assert _full({"type": "object"}, '{"anything":{"goes":[true,false]}}')
    tree = {"$defs": {"node": {"type": "object", "properties": {"v": {"type": "integer"},
                                                                   "kids": {"type": "array", "items": {"$ref": "#/$defs/node"}}},
                               "required": ["v"]}},
            "$ref": "#/$defs/node"}
    assert _full(tree, '{"v":1,"kids":[{"v":2},{"v":3,"kids":[]}]}')
    assert not _full(tree, '{"v":1,"kids":[{"w":2}]}')
    alt = {"anyOf": [{"type": "string"}, {"type": "array", "items": {"type": "integer"}, "minItems": 1}]}
    assert _full(alt, '"x"') and _full(alt, "[1,2]") and not _full(alt, "[]") and not _full(alt, "{}")
    m = JsonSchemaMatcher({"type": "string"})
    assert m.advance('"' + " " * 3) and not m.accepts("\n")          # control characters need an escape
    ws = JsonSchemaMatcher({"type": "array"})
    assert ws.advance("[") and ws.advance("  ") and not ws.accepts(" ")         # whitespace runs are bounded
    big = JsonSchemaMatcher({"type": "array", "items": {"type": "integer"}})
    assert big.advance("[" + "9" * 24) and not big.accepts("9") and big.accepts(",")   # and so are digit runs


def _byte_vocab():
    return lambda i: chr(i) if 32 <= i < 127 or i == 10 else None


def test_token_chooser_takes_the_best_valid_candidate():
    m = JsonSchemaMatcher({"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["a"]})
    ch = TokenChooser(_byte_vocab(), eos_ids=(0,))
    logits = torch.full((256,), -10.0)
    logits[ord("x")] = 5.0         # best token, not valid JSON here
    logits[ord("{")] = 1.0
    assert ch.choose(m, logits) == ord("{")
    m.advance("{")
    logits[ord('"')] = 0.5
    assert ch.choose(m, logits) == ord('"')        # '{' again is invalid, 'x' too
    assert m.advance('"a":5}') and m.done
    assert ch.choose(m, logits) == 0               # complete: end of sequence
    # with a temperature only valid candidates are drawn
    m2 = JsonSchemaMatcher({"type": "boolean"})
    import random

    got = {ch.choose(m2, logits * 0, temperature=1.0, rng=random.Random(s)) for s in range(40)}
    assert got == {ord("t"), ord("f")}


def test_engine_generates_documents_that_fit_the_schema():
    """A random-init model knows nothing about JSON: whatever it prefers, the reply of a constrained request
    parses and validates, ends when the document is complete, and unconstrained requests of the same batch are
    untouched."""
    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.frontend.openai_api import sampling_params_from_body
    from parallax_b200.frontend.tokenizer import TokenizerWrapper
    from parallax_b200.models.config import config_from_hf

    cfg = config_from_hf(dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=128,
                              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                              intermediate_size=256, vocab_size=258, tie_word_embeddings=True, rope_theta=1e4))
    tok = TokenizerWrapper(None, vocab_size=258)
    schema = {"type": "object",
              "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"},
                             "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "maxItems": 3}},
              "required": ["ok", "n"]}
    kw = dict(device="cpu", num_blocks=64, page_size=16, max_batch_size=4, chunked_prefill_size=32, seed=0)
    eng = Engine(cfg, tokenizer=tok, **kw)
    body = {"max_tokens": 200, "temperature": 0.0,
            "response_format": {"type": "json_schema", "json_schema": {"name": "x", "schema": schema}}}
    sp = sampling_params_from_body(body)
    assert json.loads(sp.json_schema) == schema
    free_sp = SamplingParams(max_new_tokens=12, temperature=0.0, ignore_eos=True)
    prompts = [tok.encode("give me json", add_special_tokens=False), tok.encode("and again", add_special_tokens=False)]
    reqs = [Request(input_ids=prompts[0], sampling_params=sp),
            Request(input_ids=prompts[1], sampling_params=SamplingParams.from_dict(dict(sp.to_dict(), temperature=0.9))),
            Request(input_ids=prompts[0], sampling_params=free_sp)]
    for r in reqs:
        eng.add_request(r)
    while eng.has_work():
        eng.step()
    from parallax_b200.engine.structured import JsonSchemaMatcher

    for r in reqs[:2]:
        text = tok.decode(r.output_ids)
        doc = json.loads(text)
        m = JsonSchemaMatcher(schema)
        assert m.advance(text) and m.done, text
        assert isinstance(doc["ok"], bool) and isinstance(doc["n"], int)
        assert r.status.name == "FINISHED_EOS" and len(r.output_ids) < 200
    want = Engine(cfg, **kw).generate([prompts[0]], free_sp)[0]
    assert reqs[2].output_ids == want
    with pytest.raises(ValueError, match="tokenizer"):
        Engine(cfg, **kw).add_request(Request(input_ids=prompts[0], sampling_params=sp))
    assert sampling_params_from_body({"response_format": {"type": "json_object"}}).json_schema == '{"type": "object"}'
    assert sampling_params_from_body({}).json_schema is None
