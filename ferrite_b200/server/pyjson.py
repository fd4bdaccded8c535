"""JSON text exactly as Python's `json.dumps` writes it (separators, escapes, key order): chat templates embed tool
schemas and arguments with `tojson`, and a byte-exact prompt needs byte-exact JSON. The reference re-implements
this in Rust (`crates/fe-server/src/pyjson.rs`); here it is the standard library itself, kept behind one name so
every caller uses the same settings."""
import json
from typing import Any


def dumps(obj: Any, indent=None, ensure_ascii: bool = False, sort_keys: bool = False) -> str:
    return json.dumps(obj, indent=indent, ensure_ascii=ensure_ascii, sort_keys=sort_keys)
