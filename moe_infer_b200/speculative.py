"""Speculative decoding with the MTP block as the drafter and a two-token verify, greedy and lossless.

The reference measures only the ceiling of this scheme: ``moe_infer/helpers/bench_mtp.py:87-126`` compares the MTP
head's draft with the token the main model picks one step later, and ``moe_infer/generation.py:94-127``
(``generate_from_mtp``) falls back to the ordinary loop "until KV-cache consistency is handled at the engine level".
Here the engine has that consistency (``Engine.snapshot_state`` / ``restore_snapshot`` carry the conv and recurrence
states of the linear-attention layers), so the loop is the real one:

    t0          the token picked from the logits in hand
    draft       argmax of ``mtp_forward(t0)``: the MTP block's guess of the token after t0
    verify      ONE ``forward([t0, draft])``: row 0 gives the main model's own pick after t0, row 1 the pick after draft
    accept      pick == draft: both tokens are emitted, row 1 is the next step's logits (two tokens for one forward)
    reject      the state is rolled back to before the verify and t0 alone is run again (its logits are row 0)

The tokens are exactly those of the ordinary greedy loop (the tests compare them).  Whether it is faster depends on the
engine's two-token forward costing less than two one-token forwards; the statistics returned say how many drafts were
accepted and how many forwards ran.  The functions only use the ``Engine`` / ``Cache`` surface of ``_moe_infer_rs``
(src/python_bindings.rs:172-311), so they run against either implementation.
"""
from __future__ import annotations

import time
from typing import Any, Callable, Optional, Sequence

import numpy as np


def greedy_decode(first_logits: np.ndarray, engine: Any, cache: Any, *, max_tokens: int = 256, eos_ids: Sequence[int] = (),
                  on_token: Optional[Callable[[int], None]] = None, mtp: bool = False) -> tuple[list, dict]:
    """The ordinary loop of ``generate_from`` (moe_infer/generation.py:66-79) at temperature 0: token ids and timings."""
    t_start = time.time()
    last = np.asarray(first_logits[-1] if np.ndim(first_logits) == 2 else first_logits)
    out: list = []
    forwards = 0
    for _ in range(max_tokens):
        tok = int(np.argmax(last))
        if tok in eos_ids:
            break
        out.append(tok)
        if on_token is not None:
            on_token(tok)
        last = engine.forward(np.array([tok], np.int64), cache, mtp=mtp)[0]
        forwards += 1
    dt = time.time() - t_start
    return out, {"tokens": len(out), "seconds": dt, "tok_per_s": len(out) / dt if out and dt > 0 else 0.0, "forwards": forwards}


def speculative_decode(first_logits: np.ndarray, engine: Any, cache: Any, *, max_tokens: int = 256, eos_ids: Sequence[int] = (),
                       on_token: Optional[Callable[[int], None]] = None) -> tuple[list, dict]:
    """Greedy decoding, one MTP draft per step, verified by a two-token forward.  Returns (token ids, statistics):
    ``drafted`` / ``accepted`` drafts, ``forwards`` of the main model and the tokens they ran, ``mtp_steps``."""
    t_start = time.time()
    last = np.asarray(first_logits[-1] if np.ndim(first_logits) == 2 else first_logits)
    out: list = []
    st = {"drafted": 0, "accepted": 0, "forwards": 0, "forward_tokens": 0, "mtp_steps": 0}

    def emit(tok: int) -> None:
        out.append(tok)
        if on_token is not None:
            on_token(tok)

    while len(out) < max_tokens:
        t0 = int(np.argmax(last))
        if t0 in eos_ids:
            break
        emit(t0)
        if len(out) >= max_tokens:
            # nothing left to draft for; keep the engine's position in step with the emitted tokens
            last = engine.forward(np.array([t0], np.int64), cache, mtp=True)[0]
            st["forwards"] += 1
            st["forward_tokens"] += 1
            break
        draft_logits = engine.mtp_forward(t0)
        st["mtp_steps"] += 1
        if np.size(draft_logits) == 0:
            raise RuntimeError("the engine has no MTP block: mtp_forward returned nothing")
        draft = int(np.argmax(draft_logits))
        st["drafted"] += 1
        snap = engine.snapshot_state()
        pos_before = cache.pos
        both = engine.forward(np.array([t0, draft], np.int64), cache, mtp=True)
        st["forwards"] += 1
        st["forward_tokens"] += 2
        pick = int(np.argmax(both[0]))
        if pick == draft and draft not in eos_ids:
            st["accepted"] += 1
            emit(draft)
            last = both[1]
            continue
        # rejected (or the draft would end the sequence): back to the state before the verify, then t0 alone
        engine.restore_snapshot(snap)
        cache.pos = pos_before
        last = engine.forward(np.array([t0], np.int64), cache, mtp=True)[0]
        st["forwards"] += 1
        st["forward_tokens"] += 1
    dt = time.time() - t_start
    st.update({"tokens": len(out), "seconds": dt, "tok_per_s": len(out) / dt if out and dt > 0 else 0.0,
               "accept_rate": st["accepted"] / st["drafted"] if st["drafted"] else 0.0})
    return out, st
