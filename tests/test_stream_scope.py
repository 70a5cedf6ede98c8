"""lib.stream_scope(): one look-up of the current stream for all launches inside, nested scopes, and the
look-up per launch outside of any scope.  No GPU: torch's look-up is replaced by a counter."""
import types

import torch

from transformer_b200.csrc import lib


def test_scope_looks_up_once_and_restores(monkeypatch):
    calls = []

    def current_stream():
        calls.append(1)
        return types.SimpleNamespace(cuda_stream=100 + len(calls))

    monkeypatch.setattr(torch.cuda, "current_stream", current_stream)
    assert lib._stream() == 101 and lib._stream() == 102, "outside a scope every launch asks torch"
    with lib.stream_scope():
        assert lib._stream() == 103 and lib._stream() == 103 and len(calls) == 3
        with lib.stream_scope():                       # e.g. a capture inside: its own stream
            assert lib._stream() == 104 and len(calls) == 4
        assert lib._stream() == 103, "the outer scope's stream is back"
    assert lib._stream() == 105, "and none after the scope"


def test_scope_ends_when_the_body_raises(monkeypatch):
    monkeypatch.setattr(torch.cuda, "current_stream", lambda: types.SimpleNamespace(cuda_stream=7))
    try:
        with lib.stream_scope():
            raise ValueError("inside")
    except ValueError:
        pass
    assert lib._scope_stream is None
