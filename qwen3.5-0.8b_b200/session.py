"""Resident session over one request state: the reference's line protocol for multi-turn decoding.

Mirrors `session_loop` of the reference driver (engine/decode_run.cpp:1760-1795, 2436-2560) and the
stop rule of engine/decode_step.h:487-492: weights and the request state stay resident across
turns; one command per line:

    feed <id> <id>...  advance the state over the caller's tokens as ONE prefill wave (only the last
                       row's logits are priced).  The token the previous turn handed to the caller
                       but never consumed (the stop token that ended it) is fed first.
                       -> "FED n=<k> prefix_len=<P>"
    gen <n>            at most n tokens, "GEN <id> <pos>" each (pos = position of the row that decided
                       the token), then "END steps=<k> stop=<0|1> prefix_len=<P>".  The stop id
                       (248046) is emitted and ends the turn.
    reset              fresh request -> "RESET prefix_len=0"
    stats              "PREFIX p=<P> sampled=<id> stopped=<0|1>"
    quit | bye         "BYE"

A failed step poisons the session until `reset` (the state is half-advanced and no longer matches
the caller's transcript).  `suspend()` / `resume()` move the request out of and back into the
engine in the reference's state-tuple layouts (engine/state.h:83-111), which is how a request is
pre-empted and resumed or migrated to another GPU.
"""
from __future__ import annotations

import torch

from .engine import Engine, LaneState, Q35Error

STOP_TOKEN = 248046          # end-of-turn id (engine/decode_step.h:492)


class Session:
    def __init__(self, engine: Engine, cap: int = 4096, stop_token: int = STOP_TOKEN):
        self.engine, self.cap, self.stop_token = engine, cap, stop_token
        self.device = getattr(engine, "device", "cuda")     # test doubles of the engine may live on the CPU
        self.state: LaneState = engine.allocate_state(1, cap)
        self.sampled_token = -1      # sampled and not yet consumed by a step (-1: none)
        self.stopped = False
        self.poisoned = False
        self._prefix = 0

    # ---- state ---------------------------------------------------------------------------------
    @property
    def prefix_len(self) -> int:
        return self._prefix

    def close(self):
        self.state.close()

    def suspend(self) -> dict:
        """The request as the reference's state tuple plus the session's own scalars."""
        blob = self.state.export_lane(0, self.cap)
        blob.update(sampled_token=self.sampled_token, stopped=self.stopped)
        return blob

    def resume(self, blob: dict) -> None:
        self.state.import_lane(0, blob["gdn_state"], blob["conv_window"], blob["kv_keys"], blob["kv_values"],
                               blob["prefix_len"])
        self._prefix = int(blob["prefix_len"])
        self.sampled_token = int(blob["sampled_token"])
        self.stopped, self.poisoned = bool(blob["stopped"]), False

    # ---- commands ------------------------------------------------------------------------------
    def reset(self) -> str:
        self.state.reset()
        self.sampled_token, self.stopped, self.poisoned, self._prefix = -1, False, False, 0
        return "RESET prefix_len=0"

    def feed(self, ids) -> str:
        tokens = ([self.sampled_token] if self.sampled_token >= 0 else []) + [int(t) for t in ids]
        if not tokens:
            raise Q35Error(1, "feed needs at least one token")
        vocab = self.engine.vocab
        for t in tokens:
            if t < 0 or t >= vocab:
                raise Q35Error(1, f"token id {t} out of range [0, {vocab})")
        dev = torch.tensor([tokens], dtype=torch.int32, device=self.device)
        y0, _ = self.engine.prefill(self.state, dev)
        self._prefix += len(tokens)
        self.sampled_token = int(y0.item())
        self.stopped = False
        return f"FED n={len(tokens)} prefix_len={self._prefix}"

    def gen(self, budget: int):
        """Yields the protocol lines of one `gen` command."""
        emitted, stop = 0, False
        cur = self.sampled_token
        tok = torch.empty(1, dtype=torch.int32, device=self.device)
        while emitted < budget:
            yield f"GEN {cur} {self._prefix - 1}"
            emitted += 1
            if cur == self.stop_token:
                stop = True
                break
            tok.fill_(cur)
            out = self.engine.decode_step(self.state, tok)
            self._prefix += 1
            cur = int(out.item())
        # a stop token was handed to the caller but never consumed: the next feed starts with it;
        # after a spent budget the last token handed out HAS been consumed and nothing is pending
        self.sampled_token = cur if stop else -1
        self.stopped = stop
        yield f"END steps={emitted} stop={1 if stop else 0} prefix_len={self._prefix}"

    def stats(self) -> str:
        return f"PREFIX p={self._prefix} sampled={self.sampled_token} stopped={1 if self.stopped else 0}"

    # ---- the line protocol ---------------------------------------------------------------------
    def handle(self, line: str):
        """Protocol lines answering one command line (empty for a blank line); 'BYE' ends the session."""
        words = line.split()
        if not words:
            return
        cmd = words[0]
        if cmd in ("quit", "bye"):
            yield "BYE"
            return
        if cmd == "reset":
            yield self.reset()
            return
        if self.poisoned:
            yield "ERROR session is poisoned by the failed step: send reset before the next feed or gen"
            return
        if cmd == "gen" and self.sampled_token < 0:
            yield "ERROR gen with no sampled token: feed this turn's prompt first"
            return
        if cmd == "gen":
            try:
                budget = int(words[1])
            except (IndexError, ValueError):
                yield "ERROR gen needs a token count"
                return
        try:
            if cmd == "feed":
                ids = []
                for w in words[1:]:
                    try:
                        ids.append(int(w))
                    except ValueError:
                        break                      # the reference stops reading ids at the first non-number
                yield self.feed(ids)
            elif cmd == "gen":
                yield from self.gen(budget)
            elif cmd == "stats":
                yield self.stats()
            else:
                yield f"ERROR unknown command: {cmd}"
        except (Q35Error, RuntimeError) as e:
            self.poisoned = True
            yield f"ERROR {e}"

    def loop(self, lines, write) -> None:
        """Serve commands from an iterable of lines, writing each answer line through `write`."""
        write(f"READY cap={self.cap}")
        for line in lines:
            for out in self.handle(line):
                write(out)
                if out == "BYE":
                    return
