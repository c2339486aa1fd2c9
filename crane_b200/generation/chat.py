"""The Hunyuan chat template, as text.

The reference formats a conversation itself rather than through the tokenizer's
template (crane/src/llm/client.rs:299-336): the begin-of-sentence mark; a leading
system message followed by a separator; then every user message behind the user
mark and every assistant message behind the assistant mark and closed by the
end mark; other roles are dropped; at the end the assistant mark, after which
the model answers.  The text is then encoded with special tokens
(crane-core/src/models/hunyuan_dense/model.rs:166-176).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

BOS = "<｜hy_begin▁of▁sentence｜>"
USER = "<｜hy_User｜>"
ASSISTANT = "<｜hy_Assistant｜>"
EOS = "<｜hy_place▁holder▁no▁2｜>"
SEP = "<｜hy_place▁holder▁no▁3｜>"


def apply_chat_template(messages: Sequence[Dict[str, str]]) -> str:
    """messages: dicts with ``role`` ("system", "user", "assistant"; anything
    else is left out) and ``content``.  Only a system message that comes first
    counts as one."""
    out = [BOS]
    rest = list(messages)
    if rest and rest[0].get("role") == "system":
        out += [rest[0]["content"], SEP]
        rest = rest[1:]
    for m in rest:
        if m.get("role") == "user":
            out += [USER, m["content"]]
        elif m.get("role") == "assistant":
            out += [ASSISTANT, m["content"], EOS]
    out.append(ASSISTANT)
    return "".join(out)


def format_chat(user_message: str, system: Optional[str] = None) -> str:
    """One user message (and an optional system message) as a prompt
    (hunyuan_dense/model.rs:178-190)."""
    msgs = ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": user_message}]
    return apply_chat_template(msgs)
