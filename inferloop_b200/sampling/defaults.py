"""Generation defaults of a model folder, and how a request's own fields override them.

The reference reads `generation_config.json` beside `config.json`
(crates/model/package/src/generation/read.rs:9-100): `do_sample` decides whether the base
temperature is 1 or 0 (absent: the provider's policy, which without a recognised model
card is "do not sample"); `temperature`, `top_p`, `min_p`, `presence_penalty`,
`repetition_penalty` and `top_k` (0 = none) are taken when present; a `do_sample` of false
forces the temperature to 0 whatever the file says; the stop tokens are `eos_token_id` of
generation_config.json, else of config.json (of its `text_config` if it has one), a number
or a list.  A request then overrides field by field
(crates/model/package/src/generation/mod.rs:68-128): `eos_tokens` replaces the list,
`eos_token` replaces it by one token, `do_sample` false forces greedy, `do_sample` true
with no temperature anywhere means temperature 1.  The model-card presets of the reference
(thinking and non-thinking chat modes) belong to its chat front end and are not read here.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict, Mapping, Optional

from .params import SamplingParams

MAX_BYTES = 1 << 20        # bounded read, as for config.json

_FLOAT_FIELDS = ("temperature", "top_p", "min_p", "presence_penalty", "repetition_penalty")
_OVERRIDES = set(_FLOAT_FIELDS) | {"top_k", "seed", "do_sample", "eos_tokens", "eos_token"}


def _read_json(path: str) -> Dict[str, Any]:
    if not os.path.exists(path):
        return {}
    if os.path.getsize(path) > MAX_BYTES:
        raise ValueError(f"{path}: larger than {MAX_BYTES} bytes")
    with open(path, "r", encoding="utf-8") as fh:
        try:
            data = json.load(fh)
        except (json.JSONDecodeError, RecursionError) as e:
            raise ValueError(f"{path}: malformed JSON: {e}") from None
    if not isinstance(data, dict):
        raise ValueError(f"{path}: not a JSON object")
    return data


def _token(value: Any) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or not (0 <= value < (1 << 32)):
        raise ValueError("invalid EOS token")
    return value


class GenerationDefaults:
    """`base` is what a request with no sampling fields gets; `sources` says where each
    field came from (the reference reports the same map)."""

    def __init__(self, base: Optional[SamplingParams] = None, sources: Optional[Dict[str, str]] = None) -> None:
        self.base = base or SamplingParams()
        self.sources = dict(sources or {})

    @classmethod
    def from_folder(cls, folder: str) -> "GenerationDefaults":
        return cls.from_configs(_read_json(os.path.join(folder, "config.json")),
                                _read_json(os.path.join(folder, "generation_config.json")))

    @classmethod
    def from_configs(cls, config: Mapping[str, Any], generation: Optional[Mapping[str, Any]] = None) -> "GenerationDefaults":
        generation = generation or {}
        fields: Dict[str, Any] = {}
        sources = {k: "runtime fallback" for k in _FLOAT_FIELDS + ("top_k", "seed", "eos_tokens")}
        sampling = False
        if "do_sample" in generation:
            if not isinstance(generation["do_sample"], bool):
                raise ValueError("do_sample must be boolean")
            sampling = generation["do_sample"]
        fields["temperature"] = 1.0 if sampling else 0.0
        for key in _FLOAT_FIELDS:
            if key in generation:
                v = generation[key]
                if isinstance(v, bool) or not isinstance(v, (int, float)):
                    raise ValueError(f"generation_config.json: {key} must be a number")
                fields[key] = float(v)
                sources[key] = "generation_config.json"
        if not sampling:
            fields["temperature"] = 0.0
            if "do_sample" in generation:
                sources["temperature"] = "generation_config.json do_sample=false"
        if "top_k" in generation:
            k = generation["top_k"]
            if isinstance(k, bool) or not isinstance(k, int) or k < 0:
                raise ValueError("invalid top_k")
            fields["top_k"] = k or None
            sources["top_k"] = "generation_config.json"
        text = config.get("text_config") if isinstance(config.get("text_config"), dict) else config
        eos = generation.get("eos_token_id", text.get("eos_token_id"))
        if eos is not None:
            fields["eos_tokens"] = tuple(_token(v) for v in (eos if isinstance(eos, list) else [eos]))
            sources["eos_tokens"] = "generation_config.json" if "eos_token_id" in generation else "config.json"
        return cls(SamplingParams(**fields), sources)

    def resolve(self, overrides: Optional[Mapping[str, Any]] = None) -> SamplingParams:
        """The base with a request's fields applied one by one."""
        o = dict(overrides or {})
        extra = set(o) - _OVERRIDES
        if extra:
            raise ValueError(f"unknown sampling fields {sorted(extra)}")   # deny_unknown_fields
        f: Dict[str, Any] = {}
        for key in _FLOAT_FIELDS + ("seed",):
            if o.get(key) is not None:
                f[key] = o[key]
        if o.get("top_k") is not None:
            f["top_k"] = o["top_k"] or None
        temperature = f.get("temperature", self.base.temperature)
        if o.get("do_sample") is False:
            f["temperature"] = 0.0
        elif o.get("do_sample") is True and o.get("temperature") is None and temperature == 0.0:
            f["temperature"] = 1.0
        if o.get("eos_tokens") is not None:
            f["eos_tokens"], f["eos_token"] = tuple(_token(t) for t in o["eos_tokens"]), None
        if o.get("eos_token") is not None:
            f["eos_token"], f["eos_tokens"] = _token(o["eos_token"]), ()
        return dataclasses.replace(self.base, **f)

    def with_stop_tokens(self, params: SamplingParams) -> SamplingParams:
        """`params` as given, except that a request which names no stop token of its own
        stops at the folder's."""
        if params.eos_token is None and not params.eos_tokens and (self.base.eos_tokens or self.base.eos_token is not None):
            return dataclasses.replace(params, eos_tokens=self.base.eos_tokens, eos_token=self.base.eos_token)
        return params
