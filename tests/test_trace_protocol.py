"""The replay program's protocol with a scripted engine in place of the GPU one: what it reads,
what it writes, and when it gives slots back (no GPU)."""
from __future__ import annotations

import io
import json

import numpy as np
import torch

import longbow_quarrel_b200  # noqa: F401
from longbow_quarrel_b200 import trace


class ScriptedEngine:
    """Logits that name their place: row = [slot, number of tokens the slot held before, place, 0...]."""
    VOCAB = 6
    made = []

    def __init__(self, **kw):
        self.kw, self.length, self.free, self.log = kw, {}, [2, 1, 0], []
        ScriptedEngine.made.append(self)

    @classmethod
    def from_pretrained(cls, folder, dtype, max_tokens):
        return cls(folder=folder, dtype=dtype, max_tokens=max_tokens)

    def new_sequence(self):
        slot = self.free.pop()
        self.length[slot] = 0
        return slot

    def end_sequence(self, slot):
        del self.length[slot]
        self.free.append(slot)
        self.log.append(("end", slot))

    def step(self, entries, want):
        assert entries, "the engine refuses a step without sequences"
        rows = []
        for (slot, tokens), ws in zip(entries, want):
            rows += [[slot, self.length[slot], w, 0, 0, 0] for w in ws]
            self.length[slot] += len(tokens)
        self.log.append(("step", [s for s, _ in entries]))
        return torch.tensor(rows, dtype=torch.float32) if rows else None

    def check(self):
        self.checks = getattr(self, "checks", 0) + 1

    def close(self):
        self.log.append(("close",))


def test_steps_files_and_slots(tmp_path, monkeypatch, capsys):
    import longbow_quarrel_b200.engine as engine_module
    monkeypatch.setattr(engine_module, "Engine", ScriptedEngine)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}, {"id": 7, "tokens": [1], "want": [0]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": []}, {"id": 7, "tokens": [2]}], "end": [7]},
        {"step": 2, "entries": [], "end": ["a", "never seen"]},
        {"step": 9, "entries": [{"id": "c", "tokens": [3, 3], "want": [1]}], "end": ["c"]},
    ]
    monkeypatch.setattr("sys.stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n\n"))
    out = tmp_path / "out"
    assert trace.main(["--model", "DIR", "--dtype", "float32", "--out", str(out), "--max-tokens", "128"]) == 0
    assert capsys.readouterr().out.split("\n")[:4] == ["done 0", "done 1", "done 2", "done 9"]
    eng = ScriptedEngine.made[-1]
    assert eng.kw == dict(folder="DIR", dtype="float32", max_tokens=128)
    # wanted places in the order of the entries and of want, little-endian float32 [wanted, vocab]
    got = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, ScriptedEngine.VOCAB)
    assert got[:, :3].tolist() == [[0, 0, 0], [0, 0, 2], [1, 0, 0]]
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "9.f32"]      # nothing wanted: no file
    # request c starts after a and 7 have ended and takes a slot that was given back
    got = np.fromfile(out / "9.f32", dtype="<f4").reshape(-1, ScriptedEngine.VOCAB)
    assert got[0, 1:3].tolist() == [0, 1] and int(got[0, 0]) in (0, 1)
    assert eng.log == [("step", [0, 1]), ("step", [0, 1]), ("end", 1), ("end", 0), ("step", [int(got[0, 0])]),
                       ("end", int(got[0, 0])), ("close",)]
    assert sorted(eng.free) == [0, 1, 2]                                    # every slot came back once
    assert eng.checks == 2                                                  # after each read of a step's logits


def test_a_wait_that_gave_up_is_raised_where_the_host_reads_results():
    """The kernels with bounded waits write a code into a word of host memory; the check raises on it, names
    the library and the wait, and clears the word.  (No device wait is made to run out: the word is set here.)"""
    import ctypes

    import pytest

    from longbow_quarrel_b200.kernels import ops
    word = (ctypes.c_int * 1)(0)
    saved = dict(ops._status_words)
    ops._status_words.clear()
    ops._status_words["gemm_tc"] = word
    try:
        ops.check_status()                       # nothing recorded: no error
        word[0] = 3
        with pytest.raises(ops.KernelError, match="gemm_tc.*stage's copies.*code 3"):
            ops.check_status()
        assert word[0] == 0
        ops.check_status()
        ops._status_words["attn_prefill_tc"] = None      # a word that could not be set up is skipped
        ops.check_status()
    finally:
        ops._status_words.clear()
        ops._status_words.update(saved)
