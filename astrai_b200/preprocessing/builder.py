"""Turn JSON records into token ids and loss masks according to a declarative section list.

Behaviour follows ``astrai/preprocessing/builder.py:29-542``:
* a *section* names a record field and an action (``train`` / ``mask`` / ``$role`` = look the message role up in
  ``config.mask``; ``value`` = copy numbers); ``template: true`` renders each message of a conversation through the
  chat template, otherwise the field is plain text;
* template configs get a masked BOS token in front; text-only all-``train`` configs apply the min / max character
  filters; everything is cut to ``max_seq_len``;
* ``SingleOutputMaskBuilder`` emits ``sequence`` (+ ``loss_mask`` unless every token trains);
  ``MultiOutputMaskBuilder`` emits one output per ``input.sources`` entry (DPO / GRPO), list-valued fields keep one
  id list per element.

Implementation: every record is first turned into a *plan* of (text, trains?, add_special_tokens) units, all units of
a batch are tokenised with two batched ``encode`` calls, then the plans are assembled.  Single-record ``build`` is a
batch of one, so both paths share one code path.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

from astrai_b200.factory import BaseFactory

Plan = List[Tuple[str, bool, bool]]  # (text, trains, add_special_tokens)
Rendered = Tuple[Optional[list], Optional[list]]


def _domain_of(item: dict, domain_key: Optional[str]) -> str:
    value = item.get(domain_key, "__default__") if domain_key else "__default__"
    return value if isinstance(value, str) else "__default__"


def _trains(action: str, role: str, config) -> bool:
    if action == "$role":
        action = config.mask.get(role, config.mask_default)
    return action == "train"


class SectionRenderer:
    # -- planning ---------------------------------------------------------------------------------------------------
    @staticmethod
    def _kind(sections: list):
        has_template = any(s.get("template") for s in sections)
        text_only = not has_template and all(s["action"] == "train" for s in sections)
        return has_template, text_only

    def _plan(self, item: dict, sections: list, config, tokenizer, text_only: bool, filter_text: bool) -> Plan:
        plan: Plan = []
        first = True
        pp = config.preprocessing
        for sec in sections:
            field, action = sec["field"], sec["action"]
            templated = sec.get("template", False)
            add_special = sec.get("add_special_tokens", not templated and first)
            if templated:
                messages = item.get(field)
                if not isinstance(messages, list) or not messages:
                    continue
                for msg in messages:
                    text = tokenizer.apply_chat_template([msg], tokenize=False, add_generation_prompt=False)
                    plan.append((text, _trains(action, msg.get("role", ""), config), False))
            else:
                text = str(item.get(field, ""))
                if not text.strip():
                    continue
                if text_only and filter_text and ((pp.min_chars > 0 and len(text) < pp.min_chars) or len(text) > pp.max_chars):
                    continue
                plan.append((text, _trains(action, "", config), add_special))
            first = False
        return plan

    # -- batched rendering --------------------------------------------------------------------------------------------
    def process_sections_batch(self, items: List[dict], sections: list, config, tokenizer, *, is_top_level=False,
                               filter_text=True) -> List[Rendered]:
        has_template, text_only = self._kind(sections)
        plans = [self._plan(it, sections, config, tokenizer, text_only, filter_text) for it in items]
        encoded = {}
        for special in (False, True):
            refs = [(i, u) for i, plan in enumerate(plans) for u, unit in enumerate(plan) if unit[2] == special]
            if refs:
                batch = tokenizer.encode([plans[i][u][0] for i, u in refs], add_special_tokens=special)
                encoded.update(zip(refs, batch))
        bos = tokenizer.bos_token_id if (is_top_level and has_template) else None
        limit = config.preprocessing.max_seq_len
        out: List[Rendered] = []
        for i, plan in enumerate(plans):
            ids, mask = ([bos], [0]) if bos is not None else ([], [])
            for u, (_, trains, _) in enumerate(plan):
                piece = encoded[(i, u)]
                ids.extend(piece)
                mask.extend([1 if trains else 0] * len(piece))
            ids, mask = ids[:limit], mask[:limit]
            empty = not ids or (is_top_level and has_template and len(ids) <= 1)
            out.append((None, None) if empty else (ids, mask))
        return out

    def process_sections(self, item: dict, sections: list, config, tokenizer, *, is_top_level=False) -> Rendered:
        return self.process_sections_batch([item], sections, config, tokenizer, is_top_level=is_top_level)[0]

    def process_list_field_batch(self, items: List[dict], sections: list, config, tokenizer) -> List[Rendered]:
        """List-valued fields (GRPO responses): one id list and one mask list per element, element order kept."""
        ids_out = [[] for _ in items]
        mask_out = [[] for _ in items]
        for sec in sections:
            field, templated = sec["field"], sec.get("template", False)
            wrapped, owner = [], []
            for i, it in enumerate(items):
                values = it.get(field)
                if not isinstance(values, list):
                    continue
                for v in values:
                    if templated and not isinstance(v, list):
                        continue
                    wrapped.append({field: v if isinstance(v, list) else str(v)})
                    owner.append(i)
            pieces = self.process_sections_batch(wrapped, [{**sec, "add_special_tokens": sec.get("add_special_tokens", False)}],
                                                 config, tokenizer, is_top_level=False, filter_text=False)
            for i, (ids, mask) in zip(owner, pieces):
                if ids:
                    ids_out[i].append(ids)
                    mask_out[i].append(mask)
        return [(a, b) if a else (None, None) for a, b in zip(ids_out, mask_out)]

    def process_list_field(self, item: dict, sections: list, config, tokenizer) -> Rendered:
        return self.process_list_field_batch([item], sections, config, tokenizer)[0]

    # -- raw values (rewards) ------------------------------------------------------------------------------------------
    @staticmethod
    def is_value_section(sections: list) -> bool:
        return len(sections) == 1 and sections[0].get("action") == "value"

    @staticmethod
    def extract_raw_value(item: dict, sections: list):
        raw = item.get(sections[0]["field"])
        if raw is None:
            return None
        return [float(v) for v in raw] if isinstance(raw, list) else [float(raw)]


class BaseMaskBuilder:
    def build(self, item: dict, config, tokenizer) -> Optional[dict]:
        return self.build_batch([item], config, tokenizer)[0]

    def build_batch(self, items: List[dict], config, tokenizer) -> List[Optional[dict]]:
        raise NotImplementedError


class MaskBuilderFactory(BaseFactory["BaseMaskBuilder"]):
    pass


@MaskBuilderFactory.register("single")
class SingleOutputMaskBuilder(BaseMaskBuilder):
    def __init__(self, renderer: Optional[SectionRenderer] = None):
        self.renderer = renderer or SectionRenderer()

    def build_batch(self, items, config, tokenizer):
        sections = config.input.sections
        if not sections:
            return [None] * len(items)
        rendered = self.renderer.process_sections_batch(items, sections, config, tokenizer, is_top_level=True)
        out = []
        for item, (ids, mask) in zip(items, rendered):
            if ids is None:
                out.append(None)
                continue
            rec = {"sequence": ids, "domain": _domain_of(item, config.output.domain_key)}
            if not all(mask):
                rec["loss_mask"] = mask
            out.append(rec)
        return out


@MaskBuilderFactory.register("multi")
class MultiOutputMaskBuilder(BaseMaskBuilder):
    def __init__(self, renderer: Optional[SectionRenderer] = None):
        self.renderer = renderer or SectionRenderer()

    def build_batch(self, items, config, tokenizer):
        sources = getattr(config.input, "sources", None)
        if not sources:
            return [None] * len(items)
        records = [{} for _ in items]
        required = {name for name, spec in sources.items() if spec.get("sections")}
        for name, spec in sources.items():
            sections = spec.get("sections") or []
            if not sections:
                continue
            if self.renderer.is_value_section(sections):
                for item, rec in zip(items, records):
                    value = self.renderer.extract_raw_value(item, sections)
                    if value is not None:
                        rec[name] = value
                continue
            mask_key = spec.get("mask_key", f"{name}_mask")
            is_list = spec.get("list_field", False)
            if is_list:
                rendered = self.renderer.process_list_field_batch(items, sections, config, tokenizer)
            else:
                rendered = self.renderer.process_sections_batch(items, sections, config, tokenizer, is_top_level=True)
            for rec, (ids, mask) in zip(records, rendered):
                if ids is None:
                    continue
                rec[name] = ids
                if is_list or "mask_key" in spec or not all(mask):
                    rec[mask_key] = mask
        return [
            {**rec, "domain": _domain_of(item, config.output.domain_key)} if required and required.issubset(rec) else None
            for item, rec in zip(items, records)
        ]


@MaskBuilderFactory.register("sectioned")
class SectionedMaskBuilder(BaseMaskBuilder):
    """``input.sources`` present -> multi-output, else single-output."""

    def __init__(self):
        self._single, self._multi = SingleOutputMaskBuilder(), MultiOutputMaskBuilder()

    def build_batch(self, items, config, tokenizer):
        chosen = self._multi if getattr(config.input, "sources", None) else self._single
        return chosen.build_batch(items, config, tokenizer)
