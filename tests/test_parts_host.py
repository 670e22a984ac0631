"""What the parts tell the engine about themselves, checked on the host (no kernel runs): which steps may be
recorded in a CUDA graph, which weights a part streams first, which norms take a hint to fetch ahead."""
import torch

from llm_steadyinfer_b200.config import config_from_dict
from llm_steadyinfer_b200.models import Model
from llm_steadyinfer_b200.parts import FeedForward, Norm, PositionEncoding
from llm_steadyinfer_b200.parts.block import Block
from tiny_configs import TINY_A, TINY_B


def test_the_llama_parts_can_be_recorded_and_a_default_part_cannot():
    for cfg in (TINY_A, TINY_B):
        m = Model(config_from_dict(cfg), torch.bfloat16, "cpu")
        assert m.capturable()
        m.blocks[-1].feed_forward = FeedForward({}, torch.bfloat16, torch.device("cpu"))     # says nothing: not capturable
        assert not m.capturable()


def test_attention_with_an_unfused_position_encoding_follows_that_encoding():
    m = Model(config_from_dict(TINY_A), torch.bfloat16, "cpu")
    mixer = m.blocks[0].mixer
    assert mixer.capturable
    mixer.position = PositionEncoding({}, torch.bfloat16, torch.device("cpu"))
    assert not mixer.capturable
    mixer.position = None
    assert mixer.capturable


def test_weights_streamed_first_are_named_for_few_rows_in_bfloat16_only():
    m = Model(config_from_dict(TINY_A), torch.bfloat16, "cpu")
    b = m.blocks[0]
    b.mixer.qkv = torch.zeros(4, 4)
    b.feed_forward.gate_up = torch.zeros(4, 4)
    assert b.mixer.streams_first(8) is b.mixer.qkv and b.feed_forward.streams_first(16) is b.feed_forward.gate_up
    assert b.mixer.streams_first(17) is None and b.feed_forward.streams_first(2048) is None
    m32 = Model(config_from_dict(TINY_A), torch.float32, "cpu")
    assert m32.blocks[0].mixer.streams_first(1) is None


def test_a_norm_is_given_the_hint_only_if_it_says_it_takes_one():
    calls = []

    class Plain(Norm):
        def forward(self, resid, delta, out, rows=None):
            calls.append(("plain", rows))

    class Hinted(Norm):
        takes_ahead = True

        def forward(self, resid, delta, out, rows=None, ahead=None):
            calls.append(("hinted", ahead))

    dev = torch.device("cpu")
    w = torch.zeros(2)
    Block.norm(Plain({}, torch.float32, dev), None, None, None, w)
    Block.norm(Hinted({}, torch.float32, dev), None, None, None, w)
    Block.norm(Hinted({}, torch.float32, dev), None, None, None, None)
    assert calls == [("plain", None), ("hinted", w), ("hinted", None)]


def test_block_arrangements_are_a_registry():
    from llm_steadyinfer_b200.parts import arrangement, register_arrangement
    import pytest
    assert callable(arrangement("pre_norm"))
    with pytest.raises(KeyError) as e:
        arrangement("sandwich")
    assert "pre_norm" in str(e.value) and "sandwich" in str(e.value)
    calls = []
    register_arrangement("host_test_order", lambda block, resid, delta, ctx, cache: calls.append(block) or "out")
    b = Block(None, None, None, None, "host_test_order")
    assert b.forward(None, None, None, None) == "out" and calls == [b] and b.capturable is False
    assert Block(None, None, None, None).capturable is True          # the built-in arrangement can be recorded
