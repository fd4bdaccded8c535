"""Chat template rendering against Hugging Face `transformers`' own renders, byte for byte (fixture written by
`python -m ferrite_b200.server.gen_template_refs`; reference `crates/fe-server/tests/template_hf.rs`)."""
import json
import os

import pytest

from ferrite_b200.server.template import ChatTemplate

FIX = os.path.join(os.path.dirname(__file__), "fixtures", "hf_template_refs.json")


def _load():
    with open(FIX) as f:
        return json.load(f)


def test_renders_equal_the_transformers_reference():
    ref = _load()
    tpl = {k: ChatTemplate(v) for k, v in ref["templates"].items()}
    n_ok = n_raise = 0
    for c in ref["cases"]:
        t = tpl[c["template"]]
        if "raises" in c:
            with pytest.raises(Exception):
                t.render(c["messages"], c["tools"], c["add_generation_prompt"], **c["kwargs"])
            n_raise += 1
            continue
        got = t.render(c["messages"], c["tools"], c["add_generation_prompt"], **c["kwargs"])
        assert got == c["expected"], (c["template"], c["conversation"], bool(c["tools"]), c["add_generation_prompt"], c["kwargs"])
        n_ok += 1
    assert n_ok >= 90 and n_raise >= 1


def test_built_in_template_is_the_fixture_template():
    """The fixture was rendered from the template this package ships: regenerate it when the template changes."""
    from ferrite_b200.server.template import DEFAULT_TEMPLATE
    assert _load()["templates"]["default"] == DEFAULT_TEMPLATE
