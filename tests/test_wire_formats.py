"""Engine-core msgpack protocol and the node-to-node stage packet format."""

import msgpack
import pytest
import torch

from parallax_b200.engine.request import IntermediateRequest, Request, RequestStatus, SamplingParams
from parallax_b200.frontend import engine_core_protocol as ecp
from parallax_b200.p2p import message_util as mu


def _add_payload(**over):
    sp = {"max_tokens": 7, "min_tokens": 1, "temperature": 0.5, "top_p": 0.9, "top_k": 20, "min_p": 0.0,
          "stop_token_ids": [3, 4], "_eos_token_id": 2,
          "extra_args": {ecp.PARALLAX_ROUTING_TABLE_EXTRA_ARG: ["a", "b"],
                         ecp.PARALLAX_SCHEDULER_REQUEST_ID_EXTRA_ARG: "sched-1"}}
    sp.update(over.pop("sampling", {}))
    arr = ["rid-1", [1, 2, 3], None, sp, None, 12.5, None, None, None]
    return arr


def test_add_request_array_and_map_forms():
    req = ecp.engine_core_request_to_initial_request(msgpack.packb(_add_payload()), max_sequence_length=8)
    assert isinstance(req, Request)
    assert req.request_id == "rid-1" and req.input_ids == [1, 2, 3]
    assert req.routing_table == ["a", "b"] and req.scheduler_request_id == "sched-1"
    sp = req.sampling_params
    assert (sp.max_new_tokens, sp.min_new_tokens, sp.top_k, sp.ignore_eos) == (7, 1, 20, False)
    assert sp.stop_token_ids == {3, 4}
    assert req.max_total_length == 8  # clamped by max_sequence_length
    as_map = {"request_id": "m", "prompt_token_ids": [5], "sampling_params": None}
    r2 = ecp.engine_core_request_to_initial_request(as_map)
    assert r2.request_id == "m" and r2.sampling_params.max_new_tokens == 128
    d = ecp.decode_engine_core_request(msgpack.packb(_add_payload()))
    assert d["client_index"] == 0 and d["resumable"] is False and len(d) == 20


@pytest.mark.parametrize("field", ["logprobs", "logit_bias", "structured_outputs", "allowed_token_ids"])
def test_unsupported_sampling_fields_are_rejected(field):
    with pytest.raises(ecp.UnsupportedEngineCoreField):
        ecp.engine_core_request_to_initial_request(_add_payload(sampling={field: 1}))


def test_unsupported_request_fields_and_frames():
    p = _add_payload()
    p[2] = [{"image": 1}]
    with pytest.raises(ecp.UnsupportedEngineCoreField):
        ecp.engine_core_request_to_initial_request(p)
    with pytest.raises(ecp.UnsupportedEngineCoreField):
        ecp.engine_core_request_to_initial_request(_add_payload(sampling={"extra_args": {"foo": 1}}))
    with pytest.raises(ecp.UnsupportedEngineCoreField):
        ecp.decode_engine_core_frame(ecp.REQUEST_TYPE_UTILITY, b"")
    with pytest.raises(ValueError):
        ecp.decode_engine_core_frame(b"\x09", b"")
    kind, ids = ecp.decode_engine_core_frame(ecp.REQUEST_TYPE_ABORT, ecp.encode_engine_core_abort(["x", "y"]))
    assert kind == "abort" and ids == ["x", "y"]
    with pytest.raises(ValueError):
        ecp.decode_engine_core_request(list(range(21)))


def test_outputs_layout_and_finish_reasons():
    out = ecp.make_engine_core_output(request_id="r", new_token_ids=[9], finish_reason=ecp.EngineCoreFinishReason.LENGTH)
    assert len(out) == 13 and out[0] == "r" and out[1] == [9] and out[5] == 1 and out[12] == 0
    outs = msgpack.unpackb(ecp.encode_engine_core_outputs([out], finished_requests=["r"], timestamp=1.0))
    assert len(outs) == 8 and outs[0] == 0 and outs[3] == 1.0 and outs[5] == ["r"]
    ready = msgpack.unpackb(ecp.engine_core_ready_payload(max_model_len=4096, dtype="bfloat16", num_gpu_blocks=10))
    assert ready["vllm_version"] == "parallax" and ready["block_size"] == 16
    r = Request(input_ids=[1])
    for st, want in [(RequestStatus.FINISHED_EOS, 0), (RequestStatus.FINISHED_MAX_LENGTH, 1),
                     (RequestStatus.FINISHED_ABORT, 2), (RequestStatus.ERROR, 3)]:
        r.status = st
        assert int(ecp.finish_reason_of(r)) == want


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.int32])
def test_tensor_round_trip(dtype):
    t = (torch.randn(3, 5) * 10).to(dtype)
    back = mu.bytes_to_tensor(mu.tensor_to_bytes(t))
    assert back.dtype == dtype and back.shape == t.shape and torch.equal(back, t)


def test_forward_request_round_trip_prefill_decode_chunked():
    sp = SamplingParams(max_new_tokens=5, temperature=0.7, top_k=3, stop_token_ids=[1, 2])
    pre = IntermediateRequest("p", 8, RequestStatus.PREFILLING, input_ids=list(range(8)),
                              hidden_states=torch.randn(8, 16).bfloat16(), routing_table=["n0", "n1"],
                              sampling_params=sp, is_chunked=True, is_last_chunk=False, chunk_start=4)
    dec = IntermediateRequest("d", 21, RequestStatus.DECODING, hidden_states=torch.randn(1, 16),
                              next_token_id=77, routing_table=["n0", "n1"], token_prob=0.25, return_probs=True,
                              output_length=3)
    blob = mu.request_to_proto([pre, dec])
    assert mu.forward_mode_of(blob) == mu.FORWARD_MODE_MIXED
    a, b = mu.proto_to_request(blob)
    assert a.request_id == "p" and a.is_prefill and a.input_ids == list(range(8))
    assert a.is_chunked and not a.is_last_chunk and a.chunk_start == 4
    assert torch.equal(a.hidden_states, pre.hidden_states) and a.hidden_states.dtype == torch.bfloat16
    assert a.sampling_params.top_k == 3 and a.sampling_params.stop_token_ids == {1, 2}
    assert b.next_token_id == 77 and b.token_prob == 0.25 and b.return_probs and b.output_length == 3
    assert b.routing_table == ["n0", "n1"] and b.input_ids is None
    assert mu.forward_mode_of(mu.request_to_proto([dec])) == mu.FORWARD_MODE_DECODE
    assert mu.proto_to_abort_request(mu.abort_request_to_proto(["x"])) == ["x"]


def test_engine_core_protocol_over_sockets(tmp_path):
    """The codec on a wire: a frontend-side client binds the two ZMQ endpoints, the engine registers, takes an
    ADD frame, streams one outputs frame per token and a finish reason; an ABORT frame ends a second request."""
    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.request import SamplingParams
    from parallax_b200.engine.service import EngineLoop
    from parallax_b200.frontend.engine_core_server import EngineCoreClient, EngineCoreServer
    from parallax_b200.models.config import named_config

    cfg = named_config("tiny")
    prompt = [5, 9, 77, 3, 250, 12]
    want = Engine(cfg, device="cpu", num_blocks=64, max_batch_size=4).generate(
        [prompt], SamplingParams(max_new_tokens=7, temperature=0.0, ignore_eos=True))[0]
    inp, out = f"ipc://{tmp_path}/in.sock", f"ipc://{tmp_path}/out.sock"
    client = EngineCoreClient(inp, out)
    loop = EngineLoop(Engine(cfg, device="cpu", num_blocks=64, max_batch_size=4))
    loop.start()
    server = EngineCoreServer(loop, inp, out, max_model_len=256, dtype="float32", num_gpu_blocks=64)
    server.start()
    try:
        info = client.wait_ready()
        assert info["max_model_len"] == 256 and info["vllm_version"] == "parallax"
        client.add("r1", prompt, {"max_tokens": 7, "temperature": 0.0})
        toks, reason = [], None
        while reason is None:
            frame = client.read(30)
            assert frame is not None, "the engine stopped answering"
            for o in frame[1]:
                assert o[0] == "r1"
                toks += o[1]
                reason = o[5] if o[5] is not None else reason
        assert toks == want and reason == 1          # finished by length
        client.add("r2", prompt, {"max_tokens": 200, "temperature": 0.0})
        assert client.read(30) is not None
        client.abort(["r2"])
        reason = None
        for _ in range(400):
            frame = client.read(30)
            assert frame is not None
            for o in frame[1]:
                if o[5] is not None:
                    reason = o[5]
            if reason is not None:
                break
        assert reason == 2                            # aborted
    finally:
        server.stop()
        loop.stop()
        client.close()
