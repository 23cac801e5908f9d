"""OpenAI-style tool definitions (JSON schema) -> the TypeScript-like declaration text that Kimi-K2.5's chat template puts in
the system turn (the job of paddleformers/transformers/kimi_k25/tool_declaration_ts.py). The text is what the model was
trained on, so its quirks are kept: Python spellings of ``None`` / ``True`` / ``False`` in enums and defaults, required fields
first and each group sorted by name, the root object's fields in declared order when a schema refers to itself."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional

INDENT = "  "
_UNION_NAMES = {"string": "string", "number": "number", "integer": "number", "boolean": "boolean", "null": "null",
                "object": "{}", "array": "Array<any>"}
_CONSTRAINTS = {"string": ("maxLength", "minLength", "pattern"), "number": ("maximum", "minimum"),
                "integer": ("maximum", "minimum"), "array": ("minItems", "maxItems")}


def _comment(text: str, indent: str = "") -> str:
    return "\n".join(f"{indent}// {line}" if line else "" for line in text.split("\n"))


class _Scope:
    """The ``$defs`` of one function and whether any ``$ref`` points at the root ('#')."""

    def __init__(self):
        self.defs: Dict[str, Any] = {}
        self.self_ref = False


def _kind(schema) -> str:
    if isinstance(schema, bool):
        return "bool"
    for key in ("$ref", "anyOf", "enum"):
        if key in schema:
            return key
    if "type" in schema:
        t = schema["type"]
        return "union" if isinstance(t, list) else t if t in ("object", "array") else "scalar"
    if schema == {}:
        return "any"
    raise ValueError(f"not a JSON schema this renderer knows: {schema}")


def _check_enum(schema):
    t = schema.get("type")
    if t is None:
        return
    if isinstance(t, list):
        rest = [x for x in t if x != "null"]
        if len(t) > 2 or (len(t) == 2 and len(rest) != 1):
            raise ValueError(f"enum of type {t} is not supported")
        t = rest[0] if rest else "null"
    want = {"string": str, "number": (int, float), "integer": int, "boolean": bool}.get(t)
    for v in schema["enum"]:
        if v is not None and want is not None and not isinstance(v, want):
            raise ValueError(f"enum value {v!r} is not of type {t}")


def _doc(schema, indent: str) -> str:
    """Comment lines above a field or an array item: its description, then its constraints sorted by name."""
    if isinstance(schema, bool):
        return ""
    kind = _kind(schema)
    lines = []
    if schema.get("description"):
        lines.append(_comment(schema["description"], indent))
    keys = _CONSTRAINTS.get(schema.get("type") if kind == "scalar" else kind, ())
    found = sorted((k, v) for k, v in schema.items() if k in keys)
    if found:
        lines.append(indent + "// " + ", ".join(f"{k}: {v}" for k, v in found))
    return "".join(line + "\n" for line in lines)


def _field(name: str, schema, optional: bool, indent: str, scope: Optional[_Scope]) -> str:
    text = _doc(schema, indent)
    default = schema.get("default") if isinstance(schema, dict) else None
    if default is not None:
        shown = repr(default) if isinstance(default, (int, float, bool)) else json.dumps(default, ensure_ascii=False)
        text += f"{indent}// Default: {shown}\n"
    return text + f"{indent}{name}{'?' if optional else ''}: {_type(schema, indent, scope)}"


def _fields(schema, indent: str, scope, in_order: bool = False) -> List[str]:
    props = schema.get("properties") or {}
    required = set(schema.get("required", []))
    names = list(props) if in_order else sorted(n for n in props if n in required) + sorted(n for n in props if n not in required)
    return [_field(n, props[n], n not in required, indent, scope) for n in names]


def _type(schema, indent: str = "", scope: Optional[_Scope] = None) -> str:
    kind = _kind(schema)
    if kind == "bool":
        return "any" if schema else "null"
    if kind == "$ref" and scope is None:                      # without a scope a reference is read by its other keys
        kind = _kind({k: v for k, v in schema.items() if k != "$ref"})
    if kind == "$ref":
        ref = schema["$ref"]
        if ref == "#":
            scope.self_ref = True
            return "parameters"
        if not ref.startswith("#/$defs/"):
            raise ValueError(f"unsupported reference: {ref}")
        name = ref.split("/")[-1]
        if name not in scope.defs:
            raise ValueError(f"reference not found: {ref}")
        return name
    if kind == "anyOf":
        return " | ".join(_type(t, indent, scope) for t in schema["anyOf"])
    if kind == "enum":
        _check_enum(schema)
        return " | ".join(f'"{e}"' if isinstance(e, str) else str(e) for e in schema["enum"])
    if kind == "union":
        return " | ".join(_UNION_NAMES[t] for t in schema["type"])
    if kind == "any":
        return "any"
    if kind == "scalar":
        return "number" if schema["type"] == "integer" else schema["type"]
    if kind == "array":
        item = schema.get("items") or {}
        doc = _doc(item, indent + INDENT)
        if doc:
            return "Array<\n" + doc + indent + INDENT + _type(item, indent + INDENT, scope) + "\n" + indent + ">"
        return f"Array<{_type(item, indent, scope)}>"
    return _object(schema, indent, scope)


def _object(schema, indent: str, scope: Optional[_Scope]) -> str:
    if scope is not None and schema.get("$defs"):
        scope.defs.update(schema["$defs"])
    rows = _fields(schema, indent + INDENT, scope)
    extra = schema.get("additionalProperties")
    if extra is not None:
        shown = "any" if extra is True else "never" if extra is False else _type(extra, indent + INDENT, scope)
        rows.append(f"{indent + INDENT}[k: string]: {shown}")
    return "{\n" + ",\n".join(rows) + "\n" + indent + "}" if rows else "{}"


def function_to_typescript(function: Dict[str, Any]) -> str:
    """One ``{"name", "description", "parameters"}`` definition -> interfaces for its ``$defs`` (and for the parameter object
    itself when something refers to '#'), the description as comment lines, and ``type name = (_: {...}) => any;``."""
    scope = _Scope()
    params = function.get("parameters") or {}
    inline = _object(params, "", scope)
    blocks = []
    if scope.self_ref:
        rows = ",\n".join(_fields(params, INDENT, scope, in_order=True))
        blocks.append("interface parameters {" + (f"\n{rows}\n" if rows else "") + "}")
    for name, sub in dict(scope.defs).items():
        head = _comment(sub["description"]) + "\n" if isinstance(sub, dict) and sub.get("description") else ""
        blocks.append(f"{head}interface {name} {_type(sub, '', scope)}")
    name = function.get("name", "function")
    description = function.get("description")
    parts = ["\n".join(blocks), _comment(description) if description else "",
             f"type {name} = (_: {'parameters' if scope.self_ref else inline}) => any;"]
    return "\n".join(p for p in parts if p)


def tools_to_typescript(tools: Optional[List[Dict[str, Any]]]) -> str:
    """The '# Tools' block for a list of ``{"type": "function", "function": {...}}`` entries; other entry types are skipped.
    Empty string when there is nothing to declare."""
    functions = [function_to_typescript(t["function"]) for t in tools or [] if t.get("type") == "function" and t.get("function")]
    if not functions:
        return ""
    return "# Tools\n\n## functions\nnamespace functions {\n" + "\n".join(functions) + "\n}\n"


def sort_keys_deep(obj: Any) -> Any:
    """Dictionaries re-created with sorted keys at every depth (the chat template sees tools in a canonical order)."""
    if isinstance(obj, dict):
        return {k: sort_keys_deep(v) for k, v in sorted(obj.items())}
    if isinstance(obj, list):
        return [sort_keys_deep(v) for v in obj]
    return obj
