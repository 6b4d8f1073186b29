"""bin/trace_run driven as a user drives it: steps on standard input, one at a
time, ``done <step>`` awaited before the next, logits read from the files it
writes.  The same requests are replayed whole, with the last 32 tokens one by
one, and in batches of unequal lengths one after another through a cache sized
by --max-tokens, in float32 and in bfloat16, and compared with the plain
implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, TINY, assert_close, make_prompts

pytestmark = pytest.mark.gpu


class Replay:
    def __init__(self, model, dtype, out, max_tokens):
        self.out = str(out)
        self.proc = subprocess.Popen(
            [os.path.join(ROOT, "bin", "trace_run"), "--model", model, "--dtype", dtype,
             "--out", self.out, "--max-tokens", str(max_tokens)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.step_no = 0

    def step(self, entries, end=()):
        rec = {"step": self.step_no, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.step_no}", f"trace_run answered {line!r}"
        path = os.path.join(self.out, f"{self.step_no}.f32")
        wanted = sum(len(e.get("want", [])) for e in entries)
        self.step_no += 1
        if wanted == 0:
            assert not os.path.exists(path)
            return None
        data = np.fromfile(path, dtype="<f4")
        return data.reshape(wanted, -1)

    def close(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=60) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_every_cutting(model_folders, plain_logits, tmp_path, name, dtype):
    vocab = TINY[name]["vocab_size"]
    lengths = [40, 97, 33, 130]
    prompts = make_prompts(name, lengths, seed=21)
    want = [plain_logits(name, p) for p in prompts]
    # 4 pages: the batch of the two longest requests (2 + 3 pages) would not fit,
    # so the cache size really comes from --max-tokens
    r = Replay(model_folders[name], dtype, tmp_path / "out", max_tokens=64 * 4)
    try:
        # (1) each request alone and whole
        for i, p in enumerate(prompts):
            got = r.step([{"id": f"w{i}", "tokens": p, "want": list(range(len(p)))}], end=[f"w{i}"])
            assert got.shape == (len(p), vocab)
            assert_close(got, want[i], dtype, f"{name} {dtype} whole {i}")
        # (2) whole prefix, then the last 32 tokens one by one
        for i, p in enumerate(prompts):
            head = len(p) - 32
            rows = [r.step([{"id": f"d{i}", "tokens": p[:head], "want": [head - 1]}])]
            for t in range(head, len(p)):
                last = t == len(p) - 1
                rows.append(r.step([{"id": f"d{i}", "tokens": [p[t]], "want": [0]}],
                                   end=[f"d{i}"] if last else []))
            assert_close(np.concatenate(rows), want[i][head - 1:], dtype, f"{name} {dtype} decoded {i}")
        # (3) batches of unequal lengths, the shorter requests ending earlier, one
        # batch after another: the slots and pages of batch one serve batch two
        for batch in ([0, 2], [1, 2], [3, 0]):
            ids = {i: f"b{batch[0]}{batch[1]}_{i}" for i in batch}
            heads = {i: len(prompts[i]) - (5 if i == batch[0] else 12) for i in batch}
            rows = {i: [] for i in batch}
            got = r.step([{"id": ids[i], "tokens": prompts[i][:heads[i]], "want": [0, heads[i] - 1]}
                          for i in batch])
            for j, i in enumerate(batch):
                assert_close(got[2 * j], want[i][0], dtype, "first place")
                rows[i].append(got[2 * j + 1: 2 * j + 2])
            t = 0
            live = list(batch)
            while live:
                entries = [{"id": ids[i], "tokens": [prompts[i][heads[i] + t]], "want": [0]} for i in live]
                done = [i for i in live if heads[i] + t + 1 == len(prompts[i])]
                got = r.step(entries, end=[ids[i] for i in done])
                for j, i in enumerate(live):
                    rows[i].append(got[j:j + 1])
                live = [i for i in live if i not in done]
                t += 1
            for i in batch:
                assert_close(np.concatenate(rows[i]), want[i][heads[i] - 1:], dtype,
                             f"{name} {dtype} batch {batch} request {i}")
        # a step that wants nothing writes no file
        assert r.step([{"id": "q", "tokens": [1, 2, 3], "want": []}], end=["q"]) is None
    finally:
        r.close()
