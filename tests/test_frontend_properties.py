"""Property tests of the text path and the wire: incremental detokenisation equals one-shot decoding (whatever the
token boundaries inside multi-byte characters and wherever a stop string falls), and stage packets survive the wire."""

import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from parallax_b200.engine.request import IntermediateRequest, RequestStatus, SamplingParams
from parallax_b200.frontend.tokenizer import ByteTokenizer, IncrementalDetokenizer, TokenizerWrapper
from parallax_b200.p2p.message_util import proto_to_request, request_to_proto

TOK = TokenizerWrapper(ByteTokenizer(), vocab_size=512)
texts = st.text(alphabet=st.sampled_from(list("ab cé中🙂\n.!STOP")), max_size=40)


@settings(max_examples=200, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(texts)
def test_streamed_pieces_add_up_to_the_decoded_text(text):
    ids = TOK.encode(text, add_special_tokens=False)
    d = IncrementalDetokenizer(TOK)
    pieces = [d.add(t) for t in ids] + [d.flush()]
    assert "".join(pieces) == TOK.decode(ids) == text
    assert all("�" not in p for p in pieces)             # no piece ends inside a character


@settings(max_examples=200, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(texts, st.sampled_from(["STOP", "é中", ".", "b c", "\n\n"]))
def test_stop_strings_cut_the_stream_exactly(text, stop):
    ids = TOK.encode(text, add_special_tokens=False)
    d = IncrementalDetokenizer(TOK, stop=[stop])
    out = ""
    for t in ids:
        out += d.add(t)
        if d.stopped:
            break
    out += d.flush()
    want = text.split(stop)[0] if stop in text else text
    assert out == want and d.stopped == (stop in text)


packet = st.builds(
    dict, rid=st.text(min_size=1, max_size=12), pos=st.integers(0, 100000), prefill=st.booleans(),
    ids=st.lists(st.integers(0, 150000), max_size=20), tok=st.one_of(st.none(), st.integers(0, 150000)),
    table=st.lists(st.text(min_size=1, max_size=8), max_size=4), rows=st.integers(0, 5),
    dtype=st.sampled_from([torch.float32, torch.bfloat16, torch.float16]), prob=st.one_of(st.none(), st.floats(0, 1)),
    chunked=st.booleans(), last=st.booleans(), start=st.integers(0, 5000), lora=st.one_of(st.none(), st.just("adapter-a")),
    temp=st.floats(0, 2), top_k=st.integers(0, 50), max_new=st.integers(1, 4096), abort=st.booleans())


@settings(max_examples=150, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.lists(packet, min_size=1, max_size=4))
def test_stage_packets_survive_the_wire(specs):
    pks = []
    for s in specs:
        h = torch.randn(s["rows"], 8).to(s["dtype"]) if s["rows"] else None
        pk = IntermediateRequest(s["rid"], s["pos"], RequestStatus.PREFILLING if s["prefill"] else RequestStatus.DECODING,
                                 input_ids=s["ids"] or None, hidden_states=h, next_token_id=s["tok"], routing_table=s["table"],
                                 sampling_params=SamplingParams(max_new_tokens=s["max_new"], temperature=s["temp"], top_k=s["top_k"]),
                                 lora_path=s["lora"], token_prob=s["prob"], return_probs=s["prob"] is not None,
                                 is_chunked=s["chunked"], is_last_chunk=s["last"], chunk_start=s["start"])
        pk.abort = s["abort"]
        pks.append(pk)
    back = proto_to_request(request_to_proto(pks))
    assert len(back) == len(pks)
    for a, b in zip(pks, back):
        assert (a.request_id, a.current_position, a.status, a.input_ids, a.next_token_id, a.routing_table, a.lora_path,
                a.is_chunked, a.is_last_chunk, a.chunk_start, a.abort, a.return_probs) == \
               (b.request_id, b.current_position, b.status, b.input_ids, b.next_token_id, b.routing_table, b.lora_path,
                b.is_chunked, b.is_last_chunk, b.chunk_start, b.abort, b.return_probs)
        assert (a.token_prob is None) == (b.token_prob is None) and (a.token_prob is None or abs(a.token_prob - b.token_prob) < 1e-6)
        assert a.sampling_params.to_dict() == b.sampling_params.to_dict()
        if a.hidden_states is None:
            assert b.hidden_states is None
        else:
            assert b.hidden_states.dtype == a.hidden_states.dtype and torch.equal(a.hidden_states, b.hidden_states)
