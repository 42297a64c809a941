"""The reference's logit-rule set, compiled into the engine's rule descriptors.

``decode_batch`` (src/whisperdrz/decoding.py:971-2046) classifies every active
row on the host into constraint groups (Phase 1, :1098-1456, 1462-1512) and
then builds a ``[rows, vocab]`` blocked mask on the device with about thirty
ordered tensor operations (Phase 2, :1514-1713) before it adds -65504, applies
the repetition penalty and takes the arg-max (Phase 3, :1717-1777).  This module
is the binding between that host classification and the fused device kernel:

* ``RuleTables`` holds the reference's vocabulary class masks
  (``DecoderState.init_gpu_tensors`` :397-724) as the engine's bitset tables:
  the class masks used by Phase 2 at indices below 32 (so that a descriptor
  can OR any of them through ``table_bits``), then per-language base sets and
  the 506 tag-prefix allow lists, which descriptors name by index;
* ``row_ops`` writes down, for one row, the Phase-2 operations in the
  reference's order from the row's group memberships;
* ``fold`` turns that ordered list into the descriptor's normal form (base mode,
  OR-ed tables, allow list, blocked timestamp prefix, single ids set and
  cleared).  Single ids are resolved exactly by replaying the operations for
  those ids on the host, so an id that the reference sets and a later class
  mask covers, or clears and a later mask re-blocks, ends up as the reference
  leaves it.

``compile_rows`` = ``row_ops`` + ``fold`` for a batch, returning the int32
``[rows, 32]`` array that ``Engine.rules_argmax`` / ``decode_step`` take.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import capi
from .dims import TOK_EOT, TOK_TS_BEGIN

# Phase-2 class masks by the names ``DecoderState.get_gpu_tensor`` knows them under.
CLASS_TABLES = (
    "block_less_than", "block_angle_consecutive", "block_asterisk", "asterisk_blocked_mask",
    "block_contains_space", "block_timings", "after_timing_blocked", "block_space_starting", "block_punct",
    "block_quote", "block_contains_close_bracket", "in_angle_blocked", "space_asterisk_token",
    "block_open_bracket", "block_greater_than", "in_paren_blocked", "block_close_paren",
)
# masks that Phase 2 only ever uses as "everything except this class"
ALLOW_TABLES = ("lang_enabled", "speaker_id_mask", "space_starting_enabled")
FIRST_CLASS = 2                      # tables 0 and 1 stay the special-token and timestamp classes of ``rules.py``
FIRST_NAMED = capi.MAX_TABLES        # tables from here on are named by index only

# hard-coded ids of the reference (decoding.py:1487-1490, 1562, 1583, 1592)
ID_OPEN_BRACKET, ID_CLOSE_BRACKET, ID_SPACE_BRACKET, ID_CUT, ID_BRACKET_PAIR, ID_SPACE = 58, 60, 542, 6672, 7131, 220

# operation kinds of the ordered list
OR, OR_NAMED, OR_NOT, ALL, ALL_EXCEPT, SET, CLEAR, PREFIX, OPEN_RANGE = range(9)


@dataclass
class RuleTables:
    """Vocabulary class masks as rows of one bool matrix, plus the name -> row index."""
    n_vocab: int
    masks: list = field(default_factory=list)          # bool [V] per table
    index: dict = field(default_factory=dict)          # name -> table index
    newline_id: int = 198
    timing_ids: np.ndarray | None = None               # id of timestamp i (contiguous in the reference vocabulary)

    @classmethod
    def empty(cls, n_vocab: int) -> "RuleTables":
        t = cls(n_vocab)
        special = np.zeros(n_vocab, bool)
        special[TOK_EOT:TOK_TS_BEGIN] = True
        t._put("special", special)
        t._put("block_timings", np.zeros(n_vocab, bool))   # filled by the caller; index 1 by construction
        return t

    def _put(self, name: str, mask) -> int:
        m = np.zeros(self.n_vocab, bool)
        src = np.asarray(mask, dtype=bool)[: self.n_vocab]
        m[: len(src)] = src
        if name in self.index:
            self.masks[self.index[name]] = m
        else:
            self.index[name] = len(self.masks)
            self.masks.append(m)
        return self.index[name]

    @classmethod
    def from_decoder_state(cls, ds, allow_tags: bool = False, allow_asterisks: bool = False,
                           languages=("en",)) -> "RuleTables":
        """``ds``: the reference's ``DecoderState`` (or anything with its ``get_gpu_tensor``, ``_cpu_masks``,
        ``get_base_blocked_cpu`` and ``_single_char_ids``)."""
        V = int(ds.vocab_size)
        t = cls.empty(V)
        get = lambda name: ds.get_gpu_tensor(name).detach().cpu().numpy().astype(bool)[:V]
        t._put("block_timings", get("block_timings"))
        for name in CLASS_TABLES:
            if name not in t.index:
                t._put(name, get(name))
        if len(t.masks) > FIRST_NAMED:
            raise ValueError("more class tables than table_bits can address")
        while len(t.masks) < FIRST_NAMED:
            t.index[f"_unused{len(t.masks)}"] = len(t.masks)
            t.masks.append(np.zeros(V, bool))
        for name in ALLOW_TABLES:
            t._put(name, get(name))
        t.allow_tags, t.allow_asterisks = allow_tags, allow_asterisks
        t._angle, t._asterisk = get("angle_blocked_mask"), get("asterisk_blocked_mask")
        t._base_of = lambda lang: ds.get_base_blocked_cpu(lang).numpy().astype(bool)[:V]
        for lang in languages:
            t.base_tables(lang)
        for prefix, ids in ds._cpu_masks["bracket_allowed"].items():
            m = np.zeros(V, bool)
            ok = [i for i in ids if i < V]
            m[ok if ok else [ds._single_char_ids["]"]]] = True      # no continuation: only the closing bracket
            t._put("bracket:" + prefix, m)
        only_close = np.zeros(V, bool)
        only_close[ds._single_char_ids["]"]] = True
        t._put("bracket:__none__", only_close)                         # a prefix no tag starts with (:1631-1637)
        t.newline_id = int(ds._single_char_ids["\n"])
        t.timing_ids = np.asarray(ds._cpu_masks["timing_token_ids"], dtype=np.int64)
        if not np.array_equal(t.timing_ids, t.timing_ids[0] + np.arange(len(t.timing_ids))):
            raise ValueError("timestamp ids are not contiguous in this vocabulary")
        return t

    def base_tables(self, lang) -> tuple[int, int]:
        """(raw, effective) table indices of a language's base blocked set; effective = raw with the tag
        and emphasis tokens unblocked when the transcriber allows them (decoding.py:1533-1543)."""
        key = lang if lang and lang != "auto" else "en"
        if "base:" + key not in self.index:
            raw = self._base_of(key)
            eff = raw.copy()
            if self.allow_tags:
                eff &= ~self._angle
            if self.allow_asterisks:
                eff &= ~self._asterisk
            self._put("base:" + key, raw)
            self._put("base_eff:" + key, eff)
        return self.index["base:" + key], self.index["base_eff:" + key]

    def matrix(self) -> np.ndarray:
        return np.stack(self.masks)

    # ---- storage (the golden fixtures keep the reference's tables this way)
    def to_arrays(self) -> dict:
        names = sorted(self.index, key=self.index.get)
        return {"names": np.array(names), "bits": np.packbits(self.matrix(), axis=1, bitorder="little"),
                "n_vocab": np.int64(self.n_vocab), "newline_id": np.int64(self.newline_id),
                "timing0": np.int64(self.timing_ids[0]), "n_timings": np.int64(len(self.timing_ids)),
                "flags": np.array([self.allow_tags, self.allow_asterisks])}

    @classmethod
    def from_arrays(cls, a) -> "RuleTables":
        V = int(a["n_vocab"])
        t = cls(V)
        bits = np.unpackbits(a["bits"], axis=1, bitorder="little")[:, :V].astype(bool)
        for name, row in zip(a["names"].tolist(), bits):
            t.index[name] = len(t.masks)
            t.masks.append(row)
        t.newline_id = int(a["newline_id"])
        t.timing_ids = int(a["timing0"]) + np.arange(int(a["n_timings"]))
        t.allow_tags, t.allow_asterisks = (bool(v) for v in a["flags"])
        t._base_of = None
        return t


@dataclass
class RowRules:
    """What Phase 1 decided for one sampled row: the names of the constraint groups it is in (the reference's
    ``*_indices`` lists without the suffix) and the few per-row values Phase 2 reads."""
    groups: frozenset
    language: str | None = "en"
    last_timing: float | None = None          # contexts[i]["last_timing"], seconds
    bracket_partial: str = ""                  # text after the last '[' of the row's line
    timing_range: tuple[int, int] | None = None   # (s_idx, e_idx) of _get_timing_range_cpu for special-timing rows
    penalty_ids: tuple = ()                    # set(state.recent_tokens) for penalised rows


SPECIAL_TIMING = ("force_timing", "force_timestamp", "line_start_timing", "close_bracket_even_timing")


def row_ops(r: RowRules, t: RuleTables, timing_step: float = 0.02) -> list[tuple]:
    """The Phase-2 operations that touch this row, in the order decode_batch applies them."""
    g = r.groups
    has = g.__contains__
    cls = lambda name: (OR, t.index[name])
    raw, eff = t.base_tables(r.language)
    ops: list[tuple] = [(OR_NAMED, eff)]                                            # :1527-1543
    if t.allow_tags:
        if has("block_open_angle"): ops.append(cls("block_less_than"))
        if has("block_angle_consecutive"): ops.append(cls("block_angle_consecutive"))
    if t.allow_asterisks:
        if has("block_asterisk_combined"): ops.append(cls("block_asterisk"))
        if has("block_star_after_star"): ops.append(cls("asterisk_blocked_mask"))
        if has("block_space_in_asterisk"): ops.append(cls("block_contains_space"))
        if has("block_timing_in_asterisk"): ops.append(cls("block_timings"))
    if has("block_eot"): ops.append((SET, TOK_EOT))                                # :1556-1566
    if has("block_newline"): ops.append((SET, t.newline_id))
    if has("block_cut"): ops.append((SET, ID_CUT))
    ops.append((SET, ID_BRACKET_PAIR))
    if has("block_bracket_after_close"): ops += [(SET, ID_OPEN_BRACKET), (SET, ID_SPACE_BRACKET)]
    if has("lang"): ops += [(ALL,), (ALL_EXCEPT, t.index["lang_enabled"])]          # :1569-1571
    if has("line_start_digit"): ops += [(ALL,), (ALL_EXCEPT, t.index["speaker_id_mask"])]
    if has("last_was_timing"): ops.append(cls("after_timing_blocked"))
    if has("last_was_timing_even"):                                                  # :1584-1592
        ops += [(ALL,), (ALL_EXCEPT, t.index["space_starting_enabled"]), (OR_NAMED, raw), (SET, ID_SPACE_BRACKET)]
    if has("last_was_timing_even_first_word"): ops += [(ALL,), (CLEAR, ID_SPACE)]
    if has("last_was_timing_even_timed_tag"): ops += [(ALL,), (CLEAR, ID_SPACE), (CLEAR, t.newline_id)]
    if has("last_was_timing_odd"): ops.append(cls("block_space_starting"))
    if has("last_was_space"): ops += [cls("block_punct"), cls("block_space_starting")]
    if has("block_punct_nonalnum"): ops.append(cls("block_punct"))
    if has("block_quote"): ops.append(cls("block_quote"))
    if has("in_bracket"):                                                            # :1623-1639
        name = "bracket:" + r.bracket_partial
        ops.append((OR_NOT, t.index[name] if name in t.index else t.index["bracket:__none__"]))
    if has("not_in_bracket"): ops.append(cls("block_contains_close_bracket"))
    if has("in_angle"):
        ops += [cls("in_angle_blocked"), cls("block_asterisk"), cls("space_asterisk_token"), cls("block_open_bracket")]
    if has("not_in_angle"): ops.append(cls("block_greater_than"))
    if has("in_asterisk"): ops += [cls("block_open_bracket"), cls("block_less_than")]
    if has("in_paren"): ops.append(cls("in_paren_blocked"))
    if has("not_in_paren"): ops.append(cls("block_close_paren"))
    if has("even_timings_not_after_timing"): ops.append(cls("block_timings"))
    if has("last_char_punct_or_bracket"): ops.append(cls("block_punct"))
    if has("block_open_bracket"): ops.append(cls("block_open_bracket"))
    if has("normal") and r.last_timing is not None and r.last_timing > 0:          # :1682-1689
        end = round(r.last_timing / timing_step) + 1
        if end > 0:
            ops.append((PREFIX, min(end, len(t.timing_ids))))
    if t.allow_asterisks and has("allow_space_asterisk"):                            # :1692-1693
        ops += [(CLEAR, int(i)) for i in np.nonzero(t.masks[t.index["space_asterisk_token"]])[0]]
    if any(has(n) for n in SPECIAL_TIMING):                                          # :1698-1713
        s, e = r.timing_range if r.timing_range is not None else (0, 0)
        ops += [(ALL,), (OPEN_RANGE, int(s), int(e))]
    return ops


def simulate(ops: list[tuple], t: RuleTables, ids=None) -> np.ndarray:
    """Replays an operation list the way the reference's tensor code would: blocked flags of ``ids``
    (default: the whole vocabulary)."""
    ids = np.arange(t.n_vocab) if ids is None else np.asarray(ids, dtype=np.int64)
    m = np.zeros(len(ids), bool)
    t0 = int(t.timing_ids[0])
    for op in ops:
        k = op[0]
        if k in (OR, OR_NAMED):
            m |= t.masks[op[1]][ids]
        elif k == OR_NOT:
            m |= ~t.masks[op[1]][ids]
        elif k == ALL:
            m[:] = True
        elif k == ALL_EXCEPT:
            m &= ~t.masks[op[1]][ids]
        elif k == SET:
            m[ids == op[1]] = True
        elif k == CLEAR:
            m[ids == op[1]] = False
        elif k == PREFIX:
            m |= (ids >= t0) & (ids < t0 + op[1])
        elif k == OPEN_RANGE:
            if op[1] < op[2]:
                m[(ids >= t0 + op[1]) & (ids < t0 + op[2])] = False
    return m


def fold(ops: list[tuple], t: RuleTables) -> dict:
    """Ordered operations -> one rule dict in the descriptor's normal form.  Raises ValueError for a
    sequence the normal form cannot hold (none of the reference's reachable rows does that)."""
    start = max((i for i, op in enumerate(ops) if op[0] == ALL), default=-1)
    live = ops[start + 1:]
    rule: dict = {"mode": capi.MODE_ALL if start >= 0 else capi.MODE_OR, "table_bits": 0}
    ored = False
    for op in live:
        k = op[0]
        if k == ALL_EXCEPT:
            if rule["mode"] != capi.MODE_ALL or ored:
                raise ValueError("'everything except a class' must directly follow 'block everything'")
            rule["mode"], rule["arg0"] = capi.MODE_ALL_EXCEPT_TABLE, op[1]
        elif k == OPEN_RANGE:
            if rule["mode"] != capi.MODE_ALL or ored:
                raise ValueError("an open timestamp range must directly follow 'block everything'")
            t0 = int(t.timing_ids[0])
            rule["mode"] = capi.MODE_ALL_EXCEPT_RANGE
            rule["arg0"], rule["arg1"] = (t0 + op[1], t0 + op[2]) if op[1] < op[2] else (0, 0)
        elif k == OR:
            rule["table_bits"] |= 1 << op[1]
            ored = True
        elif k == OR_NAMED:
            if rule.get("or_table", op[1]) != op[1]:
                raise ValueError("two different named tables OR-ed into one row")
            rule["or_table"] = op[1]
            ored = True
        elif k == OR_NOT:
            if rule.get("allow_table", op[1]) != op[1]:
                raise ValueError("two different allow lists on one row")
            rule["allow_table"] = op[1]
            ored = True
        elif k == PREFIX:
            t0 = int(t.timing_ids[0])
            rule["prefix_begin"], rule["prefix_end"] = t0, max(rule.get("prefix_end", 0), t0 + op[1])
            ored = True
    # single ids: what the reference ends up with against what the tables of the descriptor give
    singles = sorted({op[1] for op in ops if op[0] in (SET, CLEAR)})
    if singles:
        want = simulate(ops, t, singles)
        have = simulate([op for op in _normal_ops(rule, t)], t, singles)
        rule["set_ids"] = [i for i, w, h in zip(singles, want, have) if w and not h]
        rule["clear_ids"] = [i for i, w, h in zip(singles, want, have) if h and not w]
        if len(rule["set_ids"]) > 6 or len(rule["clear_ids"]) > 4:
            raise ValueError("too many single ids for one descriptor")
    return rule


def _normal_ops(rule: dict, t: RuleTables) -> list[tuple]:
    """The table part of a rule dict, written as operations again (for ``simulate``)."""
    t0 = int(t.timing_ids[0])
    ops: list[tuple] = []
    mode = rule.get("mode", capi.MODE_OR)
    if mode != capi.MODE_OR:
        ops.append((ALL,))
    if mode == capi.MODE_ALL_EXCEPT_TABLE:
        ops.append((ALL_EXCEPT, rule["arg0"]))
    elif mode == capi.MODE_ALL_EXCEPT_RANGE:
        ops.append((OPEN_RANGE, rule["arg0"] - t0, rule["arg1"] - t0))
    ops += [(OR, i) for i in range(capi.MAX_TABLES) if rule.get("table_bits", 0) >> i & 1]
    if rule.get("or_table"):
        ops.append((OR_NAMED, rule["or_table"]))
    if rule.get("allow_table"):
        ops.append((OR_NOT, rule["allow_table"]))
    if rule.get("prefix_end", 0) > rule.get("prefix_begin", 0):
        ops.append((PREFIX, rule["prefix_end"] - t0))
    return ops


def compile_row(r: RowRules, t: RuleTables, penalty: bool = True) -> dict:
    rule = fold(row_ops(r, t), t)
    if penalty and r.penalty_ids and not any(n in r.groups for n in SPECIAL_TIMING):
        rule["pen_ids"] = [int(i) for i in r.penalty_ids if 0 <= int(i) < t.n_vocab][:10]
    return rule


def rows_from_decode_batch(loc: dict, rows=None, timing_ranges: dict | None = None) -> list[RowRules]:
    """``RowRules`` of the sampled rows from the local variables of the reference's ``decode_batch`` as they
    stand when its Phase 1.5 is done (decoding.py:1512): every ``*_indices`` list is a constraint group, plus the
    two derived lists that carry no suffix.  ``rows``: the batch rows wanted (default ``need_sampling``);
    ``timing_ranges``: row -> (s_idx, e_idx) of ``_get_timing_range_cpu`` for the special-timing rows (the
    reference computes them inside its Phase 2 loop, :1698-1713)."""
    groups = {k[: -len("_indices")]: set(v) for k, v in loc.items() if k.endswith("_indices") and isinstance(v, list)}
    for k in ("block_asterisk_combined", "block_bracket_after_close"):
        groups[k] = set(loc.get(k, ()))
    special = set().union(*(groups.get(n, set()) for n in SPECIAL_TIMING))
    forced_close = set(loc.get("forced_close_indices", ()))
    states, contexts, counts = loc["states"], loc["contexts"], loc["token_counts"]
    out = []
    for i in (loc["need_sampling"] if rows is None else rows):
        ctx = contexts[i]
        line = ctx.get("line", "") or ""
        pen = ()
        if i not in special and i not in forced_close and counts[i] > 0:                 # decoding.py:1734-1740
            pen = tuple(set(states[i].recent_tokens))
        out.append(RowRules(
            groups=frozenset(g for g, members in groups.items() if i in members),
            language=getattr(states[i], "language", None), last_timing=ctx.get("last_timing"),
            bracket_partial=line[line.rfind("[") + 1:] if i in groups.get("in_bracket", ()) else "",
            timing_range=(timing_ranges or {}).get(i), penalty_ids=pen))
    return out


def compile_rows(rows: list[RowRules], t: RuleTables) -> np.ndarray:
    """int32 [len(rows), 32] in ``wdz_rule_desc`` layout."""
    from .transcriber import rules_to_array
    return rules_to_array([compile_row(r, t) for r in rows])
