"""Structured output: decoding constrained to a JSON schema.

The reference carries ``json_schema`` in its sampling parameters and leaves it to the grammar backend of its
GPU engines (``src/parallax/server/sampling/sampling_params.py:8-65``, ``src/parallax/sglang/batch_info.py:43-59``).
Here the constraint is an incremental matcher over characters: a set of parser stacks (a small non-deterministic
push-down automaton built on the fly from the schema) that answers "is this text still a prefix of a valid
document?" and "is the document complete?". The engine asks it about candidate tokens in descending logit order
and takes the best one that keeps the text valid (or samples among the valid ones), so nothing of the size of
the vocabulary is computed per step.

Supported schema keywords: ``type`` (object, array, string, number, integer, boolean, null, or a list of those),
``properties`` / ``required`` / ``additionalProperties``, ``items`` / ``minItems`` / ``maxItems``, ``enum``,
``const``, ``anyOf`` / ``oneOf``, ``$ref`` into ``$defs`` / ``definitions`` (recursion allowed), ``minLength`` /
``maxLength``; ``true`` / ``{}`` accept any JSON value. Object keys are emitted in the order of ``properties``
(optional ones may be left out); undeclared keys are accepted only where ``additionalProperties`` allows them.
Other keywords (``pattern``, ``format``, numeric ranges ...) are not enforced.
"""

from __future__ import annotations

import json
from typing import Optional

_WS = " \n\t\r"
_DIGITS = "0123456789"
_HEX = "0123456789abcdefABCDEF"
_MAX_WS_RUN = 2          # a model that only emits whitespace must run out of allowed continuations
_MAX_NUM_CHARS = 24      # likewise for digits


class SchemaError(ValueError):
    pass


class JsonSchemaMatcher:
    """Incremental matcher. ``advance(text)`` consumes text (returns False and leaves the state untouched if the
    text is not a valid continuation), ``accepts(text)`` only asks, ``done`` tells whether a complete document
    has been read (only whitespace may follow)."""

    def __init__(self, schema):
        if isinstance(schema, str):
            schema = json.loads(schema)
        self.root = schema
        self._defs = {}
        if isinstance(schema, dict):
            for key in ("$defs", "definitions"):
                for name, sub in (schema.get(key) or {}).items():
                    self._defs[f"#/{key}/{name}"] = sub
        # a state is a frozenset of stacks; a stack is a tuple of frames, the innermost frame last
        self._states = frozenset([(("val", self._id(schema), False),)])       # no whitespace before the document
        self.text = ""

    # ------------------------------------------------------------------ schema table
    def _id(self, schema) -> int:
        """Schemas are referred to by index (frames stay small hashable tuples)."""
        table = self.__dict__.setdefault("_table", [])
        index = self.__dict__.setdefault("_index", {})
        key = id(schema) if isinstance(schema, (dict, list)) else ("lit", schema)
        if key not in index:
            index[key] = len(table)
            table.append(schema)
        return index[key]

    def _resolve(self, sid: int):
        s = self._table[sid]
        seen = 0
        while isinstance(s, dict) and "$ref" in s:
            ref = s["$ref"]
            if ref == "#":
                s = self.root
            elif ref in self._defs:
                s = self._defs[ref]
            else:
                raise SchemaError(f"unresolvable $ref {ref!r}")
            seen += 1
            if seen > 64:
                raise SchemaError("$ref cycle without a value")
        return s

    # ------------------------------------------------------------------ public
    @property
    def done(self) -> bool:
        return any(len(st) == 0 for st in self._states)

    @property
    def alive(self) -> bool:
        return bool(self._states)

    def accepts(self, text: str) -> bool:
        return bool(self._run(self._states, text))

    def advance(self, text: str) -> bool:
        nxt = self._run(self._states, text)
        if not nxt:
            return False
        self._states = nxt
        self.text += text
        return True

    def can_finish_with(self, text: str) -> bool:
        """Whether the document is complete after ``text``."""
        return any(len(st) == 0 for st in self._run(self._states, text))

    # ------------------------------------------------------------------ automaton
    def _run(self, states, text: str):
        for ch in text:
            nxt = set()
            for st in states:
                self._step(st, ch, nxt)
            if not nxt:
                return frozenset()
            states = nxt
        return frozenset(states)

    def _step(self, st: tuple, ch: str, out: set) -> None:
        """All successor stacks of ``st`` on character ``ch`` are added to ``out``."""
        if not st:                                   # complete document: trailing whitespace only
            if ch in _WS:
                out.add(st)
            return
        frame, rest = st[-1], st[:-1]
        kind = frame[0]
        if kind == "ws":                             # optional whitespace, bounded run, then the frame below
            if ch in _WS:
                if frame[1] < _MAX_WS_RUN:
                    out.add(rest + (("ws", frame[1] + 1),))
                return
            self._step(rest, ch, out)
        elif kind == "val":
            if ch in _WS and len(frame) > 2 and not frame[2]:
                return
            self._value(rest, frame[1], ch, out)
        elif kind == "lit":
            if ch == frame[1][0]:
                out.add(rest + ((("lit", frame[1][1:]),) if len(frame[1]) > 1 else ()))
        elif kind == "str":
            self._string(rest, frame, ch, out)
        elif kind == "num":
            self._number(rest, frame, ch, out)
        elif kind == "obj":
            self._object(rest, frame, ch, out)
        elif kind == "arr":
            self._array(rest, frame, ch, out)
        else:  # pragma: no cover
            raise AssertionError(kind)

    # ---- a value of schema `sid` starts at `ch`
    def _value(self, rest: tuple, sid: int, ch: str, out: set) -> None:
        if ch in _WS:
            out.add(rest + (("val", sid), ("ws", 1)))
            return
        s = self._resolve(sid)
        if s is True or s == {} or s is None:
            s = {}
        if s is False:
            return
        for key in ("anyOf", "oneOf"):
            if isinstance(s, dict) and key in s:
                for alt in s[key]:
                    self._value(rest, self._id(alt), ch, out)
                return
        if isinstance(s, dict) and "const" in s:
            options = [s["const"]]
        elif isinstance(s, dict) and "enum" in s:
            options = s["enum"]
        else:
            options = None
        if options is not None:
            for opt in options:
                lit = json.dumps(opt, ensure_ascii=False, separators=(",", ":"))
                if lit[0] == ch:
                    out.add(rest + ((("lit", lit[1:]),) if len(lit) > 1 else ()))
            return
        types = s.get("type") if isinstance(s, dict) else None
        if types is None:
            if isinstance(s, dict) and ("properties" in s or "required" in s):
                types = ["object"]
            elif isinstance(s, dict) and "items" in s:
                types = ["array"]
            else:
                types = ["object", "array", "string", "number", "boolean", "null"]
        elif isinstance(types, str):
            types = [types]
        for t in types:
            if t == "object" and ch == "{":
                out.add(rest + (("obj", sid, 0, 0, 0),))
            elif t == "array" and ch == "[":
                out.add(rest + (("arr", sid, 0, 0),))
            elif t == "string" and ch == '"':
                lo = int(s.get("minLength", 0)) if isinstance(s, dict) else 0
                hi = int(s.get("maxLength", -1)) if isinstance(s, dict) else -1
                out.add(rest + (("str", 0, 0, lo, hi),))
            elif t in ("number", "integer"):
                io = t == "integer"
                if ch == "-":
                    out.add(rest + (("num", 0, io, 1),))
                elif ch == "0":
                    out.add(rest + (("num", 1, io, 1),))
                elif ch in "123456789":
                    out.add(rest + (("num", 2, io, 1),))
            elif t == "boolean":
                if ch == "t":
                    out.add(rest + (("lit", "rue"),))
                elif ch == "f":
                    out.add(rest + (("lit", "alse"),))
            elif t == "null" and ch == "n":
                out.add(rest + (("lit", "ull"),))

    # ---- inside a string: ("str", mode, length, min, max); mode 0 plain, 1 after a backslash, 2-5 hex digits left + 1
    def _string(self, rest, frame, ch, out):
        _k, mode, n, lo, hi = frame
        if mode == 0:
            if ch == '"':
                if n >= lo:
                    out.add(rest)
            elif ch == "\\":
                if hi < 0 or n < hi:
                    out.add(rest + (("str", 1, n, lo, hi),))
            elif ch >= " " and (hi < 0 or n < hi):
                out.add(rest + (("str", 0, n + 1, lo, hi),))
        elif mode == 1:
            if ch in '"\\/bfnrt':
                out.add(rest + (("str", 0, n + 1, lo, hi),))
            elif ch == "u":
                out.add(rest + (("str", 5, n, lo, hi),))
        elif ch in _HEX:
            out.add(rest + (("str", mode - 1 if mode > 2 else 0, n + (1 if mode == 2 else 0), lo, hi),))

    # ---- inside a number: ("num", phase, integer_only)
    #      0 after '-', 1 a lone 0, 2 integer digits, 3 after '.', 4 fraction digits, 5 after e/E, 6 after the
    #      exponent's sign, 7 exponent digits. Phases 1, 2, 4, 7 may end: the character goes to the frame below.
    def _number(self, rest, frame, ch, out):
        _k, ph, io, n = frame
        room = n < _MAX_NUM_CHARS

        def go(phase):
            out.add(rest + (("num", phase, io, n + 1),))

        if ph == 0:
            if ch == "0":
                go(1)
            elif ch in "123456789":
                go(2)
            return
        if ph in (2, 4, 7) and ch in _DIGITS:
            if room:
                go(ph)
            return
        if ph in (1, 2) and ch == "." and not io:
            if room:
                go(3)
            return
        if ph in (1, 2, 4) and ch in "eE" and not io:
            if room:
                go(5)
            return
        if ph == 3:
            if ch in _DIGITS:
                go(4)
            return
        if ph == 5:
            if ch in "+-":
                go(6)
            elif ch in _DIGITS:
                go(7)
            return
        if ph == 6:
            if ch in _DIGITS:
                go(7)
            return
        # the number is over: whoever is below sees this character (a top-level number ends at whitespace)
        if rest:
            self._step(rest, ch, out)
        elif ch in _WS:
            out.add(())

    # ---- objects: ("obj", sid, next property index, phase, number of entries so far)
    #      phase 0: after '{' or ',' - a key or (only right after '{') '}';  1: inside the key, matching names;
    #      2: after the key - ':' ; 3: after a value - ',' or '}'
    def _props(self, sid):
        s = self._resolve(sid)
        s = s if isinstance(s, dict) else {}
        props = list((s.get("properties") or {}).items())
        required = set(s.get("required") or [])
        extra = s.get("additionalProperties", not props)       # a bare {"type": "object"} takes any keys
        return props, required, extra

    def _object(self, rest, frame, ch, out):
        _k, sid, idx, phase, count = frame[:5]
        props, required, extra = self._props(sid)
        if phase == 0 or phase == 4:                 # 4: after ',' (a key must follow)
            if ch in _WS:
                out.add(rest + (frame, ("ws", 1)))
                return
            if ch == "}" and phase == 0:
                if not any(name in required for name, _s in props[idx:]):
                    out.add(rest)
                return
            if ch == '"':
                # declared keys in order: any of the next optional ones up to and including the next required one
                names = []
                for j in range(idx, len(props)):
                    names.append((j, props[j][0]))
                    if props[j][0] in required:
                        break
                else:
                    if extra is not False:
                        names.append((-1, None))     # an undeclared key
                for j, name in names:
                    if name is None:
                        out.add(rest + (("obj", sid, len(props), 2, count, self._id(extra if extra is not True else {})),
                                        ("str", 0, 0, 1, -1)))
                    else:
                        key = json.dumps(name, ensure_ascii=False)[1:]          # name" with escapes
                        out.add(rest + (("obj", sid, j + 1, 2, count, self._id(props[j][1])), ("lit", key)))
            return
        if phase == 2:                               # the key string has just closed: ':' then the value
            if ch in _WS:
                out.add(rest + (frame, ("ws", 1)))
            elif ch == ":":
                out.add(rest + (("obj", sid, idx, 3, count + 1), ("val", frame[5])))
            return
        if phase == 3:                               # after a value
            if ch in _WS:
                out.add(rest + (frame, ("ws", 1)))
            elif ch == ",":
                more_declared = idx < len(props)
                if more_declared or extra is not False:
                    out.add(rest + (("obj", sid, idx, 4, count),))
            elif ch == "}":
                if not any(name in required for name, _s in props[idx:]):
                    out.add(rest)

    # ---- arrays: ("arr", sid, items so far, phase)  phase 0 after '[' ; 1 after a value ; 2 after ','
    def _array(self, rest, frame, ch, out):
        _k, sid, n, phase = frame
        s = self._resolve(sid)
        s = s if isinstance(s, dict) else {}
        item = self._id(s.get("items", {}) if s.get("items") is not None else {})
        lo, hi = int(s.get("minItems", 0)), s.get("maxItems")
        if ch in _WS:
            out.add(rest + (frame, ("ws", 1)))
            return
        if phase in (0, 2):
            if ch == "]" and phase == 0:
                if n >= lo:
                    out.add(rest)
                return
            if hi is None or n < int(hi):
                self._value(rest + (("arr", sid, n + 1, 1),), item, ch, out)
            return
        if ch == ",":
            if hi is None or n < int(hi):
                out.add(rest + (("arr", sid, n, 2),))
        elif ch == "]" and n >= lo:
            out.add(rest)


class TokenChooser:
    """Picks the next token of a constrained request from the step's logits: the candidates are visited in
    descending logit order (top-k first, the whole vocabulary only if none of them fits) and the first one whose
    text keeps the document valid wins; with a temperature the valid ones among the visited candidates are
    sampled instead. ``token_text(id)`` gives the text a token adds (``None`` for tokens that are not text on
    their own, e.g. half of a multi-byte character)."""

    WIDTHS = (32, 512)

    def __init__(self, token_text, eos_ids=()):
        self.token_text = token_text
        self.eos_ids = tuple(eos_ids)

    def choose(self, matcher: JsonSchemaMatcher, logits_row, temperature: float = 0.0, rng=None) -> Optional[int]:
        import torch

        if matcher.done:
            # the document is complete: end the request (EOS if the model has one)
            return self.eos_ids[0] if self.eos_ids else None
        V = logits_row.shape[-1]
        for width in self.WIDTHS + (V,):
            k = min(width, V)
            vals, idx = torch.topk(logits_row.float(), k)
            vals, idx = vals.tolist(), idx.tolist()
            ok = []
            for v, i in zip(vals, idx):
                if i in self.eos_ids:
                    continue
                t = self.token_text(i)
                if t and matcher.accepts(t):
                    ok.append((v, i))
                    if temperature <= 0.0:
                        return i
            if ok:
                import math

                m = max(v for v, _i in ok)
                w = [math.exp((v - m) / temperature) for v, _i in ok]
                r = (rng.random() if rng is not None else 0.5) * sum(w)
                acc = 0.0
                for wi, (_v, i) in zip(w, ok):
                    acc += wi
                    if acc >= r:
                        return i
                return ok[-1][1]
            if k == V:
                break
        return None
