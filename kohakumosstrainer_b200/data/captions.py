"""Caption templates: `render(row, rng) -> str`, every random choice drawn from the seeded
generator it is handed, so caption variant v of row i is fixed per (seed, i, v).

Templates and options follow the reference's caption layer
(`src/kohakumoss_data/caption/template.py:66-228`, `caption/json_text.py:48-73`,
`caption/tags.py:8-40`, `caption/gbc.py`): `tags` (keep fields, fixed head, groups, group /
tag dropout, shuffle, normalisation), `nl` (natural language with tag fallback), `mix`,
`json` (lines / json, field order and dropout) and `gbc` (a region graph rendered as text,
regions clipped to the training crop, redrawn with stronger dropout until the caption fits
the text budget). `estimate_chars(catalog)` gives the planner an upper bound per row from the
catalog's character-count columns without rendering anything.
"""

from __future__ import annotations

import json
import re

import numpy as np

from ..utils.registry import Registry

CAPTIONS = Registry("caption template")
_ESCAPE = re.compile(r"\\([()\[\]{}])")
_FIELD_CHARS = {"tags": "tags_chars", "caption_nl": "nl_chars", "artist": "artist_chars", "rating": "rating_chars"}


def split_tags(text: str, sep: str = ",") -> list[str]:
    return [t.strip() for t in text.split(sep) if t.strip()]


def normalize_tag(tag: str, underscores: bool, unescape: bool) -> str:
    if underscores:
        tag = tag.replace("_", " ")
    return _ESCAPE.sub(r"\1", tag) if unescape else tag


def build_template(spec):
    """`{"template": name, **kwargs}`, a bare name, or None (= tags)."""
    if spec is None or spec == {}:
        spec = {"template": "tags"}
    if isinstance(spec, str):
        spec = {"template": spec}
    kw = dict(spec)
    return CAPTIONS.get(kw.pop("template", "tags"))(**kw)


def _keep_values(row, keep) -> list[str]:
    out = []
    for name in keep:
        v = getattr(row, name, None)
        if v in (None, ""):
            continue
        out.extend(str(x) for x in v) if isinstance(v, (list, tuple)) else out.append(str(v))
    return out


def _col(catalog, name) -> np.ndarray:
    col = _FIELD_CHARS.get(name)
    return catalog.chars[col] if col else np.zeros(len(catalog), dtype=np.int64)


def _keep_chars(catalog, keep, sep: int) -> np.ndarray:
    out = np.zeros(len(catalog), dtype=np.int64)
    for name in keep:
        c = _col(catalog, name)
        out += c + sep * (c > 0)
    return out


@CAPTIONS.register("tags")
class TagTemplate:
    def __init__(self, keep=("artist",), keep_first: int = 0, keep_sep: str = "|||", group_sep: str = "%%", shuffle: bool = True,
                 tag_dropout: float = 0.0, group_dropout: float = 0.0, underscores: bool = True, unescape: bool = True,
                 joiner: str = ", ", prefix: str = "", suffix: str = ""):
        self.keep, self.keep_first, self.keep_sep, self.group_sep = tuple(keep), keep_first, keep_sep, group_sep
        self.shuffle, self.tag_dropout, self.group_dropout = shuffle, tag_dropout, group_dropout
        self.underscores, self.unescape = underscores, unescape
        self.joiner, self.prefix, self.suffix = joiner, prefix, suffix

    def _order(self, items: list, rng) -> list:
        if not self.shuffle or len(items) < 2:
            return items
        return [items[i] for i in rng.permutation(len(items))]

    def tag_list(self, row, rng) -> list[str]:
        tags = list(row.tags or [])
        fixed, rest = tags[: self.keep_first], tags[self.keep_first :]
        if self.keep_sep in rest:
            cut = rest.index(self.keep_sep)
            fixed, rest = fixed + rest[:cut], rest[cut + 1 :]
        groups, cur = [], []
        for t in rest:
            if t == self.group_sep:
                groups.append(cur)
                cur = []
            else:
                cur.append(t)
        groups.append(cur)
        if self.group_dropout:
            groups = [g for g in groups if rng.random() >= self.group_dropout]
        kept = []
        for g in groups:
            if self.tag_dropout:
                g = [t for t in g if rng.random() >= self.tag_dropout]
            kept.append(self._order(g, rng))
        body = [t for g in self._order(kept, rng) for t in g]
        head = _keep_values(row, self.keep) + fixed
        return [normalize_tag(t, self.underscores, self.unescape) for t in head + body]

    def render(self, row, rng) -> str:
        return self.prefix + self.joiner.join(self.tag_list(row, rng)) + self.suffix

    def estimate_chars(self, catalog) -> np.ndarray:
        return len(self.prefix) + len(self.suffix) + _keep_chars(catalog, self.keep, len(self.joiner)) + catalog.chars["tags_chars"]


@CAPTIONS.register("nl")
class NaturalTemplate:
    def __init__(self, keep=(), fallback=None):
        self.keep = tuple(keep)
        self.fallback = build_template(fallback or {"template": "tags"})

    def render(self, row, rng) -> str:
        if not row.caption_nl:
            return self.fallback.render(row, rng)
        head = _keep_values(row, self.keep)
        return ((", ".join(head) + ". ") if head else "") + row.caption_nl

    def estimate_chars(self, catalog) -> np.ndarray:
        nl = catalog.chars["nl_chars"]
        return np.where(nl > 0, _keep_chars(catalog, self.keep, 2) + nl, self.fallback.estimate_chars(catalog))


@CAPTIONS.register("mix")
class MixTemplate:
    def __init__(self, p_nl: float = 0.5, nl=None, tags=None):
        self.p_nl = p_nl
        self.nl = build_template(nl or {"template": "nl"})
        self.tags = build_template(tags or {"template": "tags"})

    def render(self, row, rng) -> str:
        if row.caption_nl and rng.random() < self.p_nl:
            return self.nl.render(row, rng)
        return self.tags.render(row, rng)

    def estimate_chars(self, catalog) -> np.ndarray:
        return np.maximum(self.nl.estimate_chars(catalog), self.tags.estimate_chars(catalog))


def _text_value(v) -> str:
    if isinstance(v, str):
        return v
    if isinstance(v, (list, tuple)):
        return ", ".join(_text_value(x) for x in v)
    if isinstance(v, dict):
        return json.dumps(v, ensure_ascii=False, sort_keys=True)
    return str(v)


@CAPTIONS.register("json")
class JsonTemplate:
    def __init__(self, fields=("artist", "rating", "tags", "caption_nl"), style: str = "lines", order=(), field_dropout: float = 0.0, keep=()):
        if style not in ("lines", "json"):
            raise ValueError(f"json style must be one of ['json', 'lines'], got {style}")
        self.fields, self.style, self.order = tuple(fields), style, tuple(order)
        self.field_dropout, self.keep = field_dropout, tuple(keep)

    def render(self, row, rng) -> str:
        data = dict(row.json or {})
        for name in self.fields:
            v = getattr(row, name, None)
            if v not in (None, "", []):
                data.setdefault(name, v)
        keys = [k for k in self.order if k in data] + sorted(k for k in data if k not in self.order)
        if self.field_dropout:
            keys = [k for k in keys if k in self.keep or rng.random() >= self.field_dropout]
        if self.style == "json":
            return json.dumps({k: data[k] for k in keys}, ensure_ascii=False)
        return "\n".join(f"{k}: {_text_value(data[k])}" for k in keys)

    def estimate_chars(self, catalog) -> np.ndarray:
        out = catalog.chars["json_chars"].copy()
        for name in self.fields:
            c = _col(catalog, name)
            out += c + (len(name) + 3) * (c > 0)
        return out


@CAPTIONS.register("gbc")
class GraphTemplate:
    """Region-graph captions. The row's `json["gbc"]` (or the source's `record(locator)`) is
    `{"short": str, "detail": str, "regions": [{"label", "text", "box": [l, t, r, b] in
    0..1, "children": [...]}]}`. Sections `tags`, `nl`, `graph` are ordered by one of the
    weighted `formats`; each section has its own dropout; region depth is cut at a drawn
    detail level; regions outside the centre crop are dropped and boxes re-expressed in the
    crop's frame; a caption longer than the budget is redrawn with stronger dropout."""

    geometric = True

    def __init__(self, formats=(("nl", "graph", "tags"),), weights=None, section_dropout=None, region_dropout: float = 0.0,
                 max_depth: int = 3, coords: bool = True, min_visible: float = 0.3, retries: int = 4, tags=None):
        self.formats = [tuple(f) for f in formats]
        w = np.asarray(weights or [1.0] * len(self.formats), dtype=np.float64)
        self.weights = w / w.sum()
        self.section_dropout = dict(section_dropout or {})
        self.region_dropout, self.max_depth, self.coords = region_dropout, max_depth, coords
        self.min_visible, self.retries = min_visible, retries
        self.tag_template = build_template(tags or {"template": "tags", "keep": ()})
        self._source, self._geometry_of, self._max_chars = None, None, 0

    def bind(self, source, geometry_of=None, max_chars: int = 0):
        self._source, self._geometry_of, self._max_chars = source, geometry_of, max_chars
        return self._render_bound

    def _record(self, row) -> dict:
        rec = (row.json or {}).get("gbc")
        if rec is None and self._source is not None and hasattr(self._source, "record"):
            rec = self._source.record(row.locator)
        return rec or {}

    def _clip(self, box, frame):
        """`box` (0..1 of the stored image) in the frame of crop `frame`; None when less than
        `min_visible` of it survives."""
        if frame is None:
            return box
        l, t, r, b = box
        fl, ft, fr, fb = frame
        il, it, ir, ib = max(l, fl), max(t, ft), min(r, fr), min(b, fb)
        area = max(r - l, 0) * max(b - t, 0)
        if ir <= il or ib <= it or area <= 0 or (ir - il) * (ib - it) / area < self.min_visible:
            return None
        fw, fh = fr - fl, fb - ft
        return [(il - fl) / fw, (it - ft) / fh, (ir - fl) / fw, (ib - ft) / fh]

    def _graph(self, regions, rng, frame, depth, level, p_drop, out):
        for reg in regions or []:
            if depth > level or (p_drop and rng.random() < p_drop):
                continue
            box = self._clip(reg.get("box", [0, 0, 1, 1]), frame)
            if box is None:
                continue
            where = " [" + ",".join(f"{v:.2f}" for v in box) + "]" if self.coords else ""
            text = reg.get("text", "")
            out.append("  " * depth + f"- {reg.get('label', 'region')}{where}" + (f": {text}" if text else ""))
            self._graph(reg.get("children"), rng, frame, depth + 1, level, p_drop, out)

    def _draw(self, row, rng, frame, strength: float) -> str:
        rec = self._record(row)
        fmt = self.formats[int(rng.choice(len(self.formats), p=self.weights))]
        level = int(rng.integers(0, self.max_depth + 1))
        parts = []
        for sec in fmt:
            p = min(1.0, self.section_dropout.get(sec, 0.0) + strength)
            if p and rng.random() < p and len(parts) + 1 < len(fmt):
                continue
            if sec == "tags" and row.tags:
                parts.append(self.tag_template.render(row, rng))
            elif sec == "nl":
                text = rec.get("detail") if level > 0 and rec.get("detail") else rec.get("short") or row.caption_nl
                if text:
                    parts.append(text)
            elif sec == "graph":
                lines: list[str] = []
                self._graph(rec.get("regions"), rng, frame, 0, level, min(1.0, self.region_dropout + strength), lines)
                if lines:
                    parts.append("\n".join(lines))
        return "\n".join(parts)

    def _render_bound(self, row, rng, row_id: int) -> str:
        frame = None
        if self._geometry_of is not None:
            g = self._geometry_of(row_id)
            l, t, r, b = g.crop_ltrb
            frame = (l / g.w, t / g.h, r / g.w, b / g.h)
        text = ""
        for attempt in range(self.retries + 1):
            text = self._draw(row, rng, frame, strength=attempt / max(1, self.retries) * 0.8)
            if not self._max_chars or len(text) <= self._max_chars:
                return text
        return text[: self._max_chars]

    def render(self, row, rng) -> str:
        return self._render_bound(row, rng, row.id)

    def estimate_chars(self, catalog) -> np.ndarray:
        return catalog.chars["json_chars"] + catalog.chars["tags_chars"] + catalog.chars["nl_chars"]


def bind_template(template, source, geometry_of=None, max_chars: int = 0):
    """`render(row, rng, row_id)` of a template over its dataset entry."""
    bind = getattr(template, "bind", None)
    if bind is not None:
        return bind(source, geometry_of, max_chars)
    return _RowOnly(template)


class _RowOnly:
    """Picklable `render(row, rng, row_id)` over a template that ignores the row id."""

    def __init__(self, template):
        self.template = template

    def __call__(self, row, rng, row_id: int) -> str:
        return self.template.render(row, rng)
