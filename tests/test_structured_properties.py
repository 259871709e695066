"""Property test of the JSON-schema matcher: for random schemas, every document generated from the schema is
accepted character by character and ends the matcher; documents of another type are refused."""

import json

from hypothesis import HealthCheck, assume, given, settings
from hypothesis import strategies as st

from parallax_b200.engine.structured import JsonSchemaMatcher

_keys = st.sampled_from(["a", "b", "name", "n", "items", "x_y", "k1"])
_text = st.text(alphabet=st.sampled_from(list("abz XYZ09_-\"\\/é中\n\t")), max_size=8)


def _leaf():
    return st.one_of(
        st.just({"type": "boolean"}), st.just({"type": "null"}), st.just({"type": "integer"}), st.just({"type": "number"}),
        st.just({"type": "string"}),
        st.lists(st.one_of(st.integers(-5, 5), st.sampled_from(["red", "green", "a b", True, None])), min_size=1, max_size=3,
                 unique_by=lambda v: json.dumps(v)).map(lambda vs: {"enum": vs}),
    )


def _extend(children):
    arr = st.tuples(children, st.integers(0, 2), st.integers(0, 3)).map(
        lambda t: {"type": "array", "items": t[0], "minItems": min(t[1], t[1] + t[2]), "maxItems": t[1] + t[2]})
    obj = st.tuples(st.dictionaries(_keys, children, min_size=1, max_size=3), st.data()).map(lambda t: t[0])
    obj = st.dictionaries(_keys, children, min_size=1, max_size=3).flatmap(
        lambda props: st.lists(st.sampled_from(sorted(props)), unique=True, max_size=len(props)).map(
            lambda req: {"type": "object", "properties": props, "required": req, "additionalProperties": False}))
    return st.one_of(arr, obj)


schemas = st.recursive(_leaf(), _extend, max_leaves=8)


@st.composite
def instance_of(draw, schema):
    if "enum" in schema:
        return draw(st.sampled_from(schema["enum"]))
    t = schema["type"]
    if t == "boolean":
        return draw(st.booleans())
    if t == "null":
        return None
    if t == "integer":
        return draw(st.integers(-10 ** 6, 10 ** 6))
    if t == "number":
        return draw(st.one_of(st.integers(-1000, 1000), st.floats(-1e6, 1e6, allow_nan=False, allow_infinity=False)))
    if t == "string":
        return draw(_text)
    if t == "array":
        n = draw(st.integers(schema.get("minItems", 0), schema.get("maxItems", 3)))
        return [draw(instance_of(schema["items"])) for _ in range(n)]
    out = {}
    for k, sub in schema["properties"].items():      # keys in the schema's order, optional ones sometimes left out
        if k in schema["required"] or draw(st.booleans()):
            out[k] = draw(instance_of(sub))
    return out


@settings(max_examples=200, deadline=None, suppress_health_check=[HealthCheck.too_slow, HealthCheck.filter_too_much])
@given(st.data())
def test_generated_documents_are_accepted_and_end_the_matcher(data):
    schema = data.draw(schemas)
    doc = data.draw(instance_of(schema))
    compact = data.draw(st.booleans())
    text = json.dumps(doc, ensure_ascii=data.draw(st.booleans()), separators=(",", ":") if compact else (", ", ": "))
    m = JsonSchemaMatcher(schema)
    for i, ch in enumerate(text):
        assert m.accepts(ch), (schema, text, i)
        assert m.advance(ch)
    top_is_number = isinstance(doc, (int, float)) and not isinstance(doc, bool)
    # a number at the top level has no closing character: it ends at the whitespace after it
    assert m.done or (top_is_number and m.can_finish_with(" ")), (schema, text)
    # the same document through one call
    m2 = JsonSchemaMatcher(schema)
    assert m2.advance(text)


@settings(max_examples=100, deadline=None, suppress_health_check=[HealthCheck.too_slow, HealthCheck.filter_too_much])
@given(st.data())
def test_documents_of_another_type_are_refused(data):
    schema = data.draw(schemas)
    assume("enum" not in schema)
    wrong = {"boolean": "1", "null": "true", "integer": '"x"', "number": "[1]", "string": "{", "array": '{"a":1}',
             "object": "[1]"}[schema["type"]]
    m = JsonSchemaMatcher(schema)
    assert not (m.advance(wrong) and m.done)
