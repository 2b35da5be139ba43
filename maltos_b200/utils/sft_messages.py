"""Turning one dataset row into SFT tokens plus a per-token supervision mask.

A row carries either a chat transcript (list of ``{"role", "content"}``, possibly JSON-encoded, content possibly a list
of text parts) or a prompt/completion pair. Tokenisation goes through the tokenizer's chat template when asked (the
template must expose ``{% generation %}`` blocks for assistant-only loss) or through a plain ``"role: text"`` rendering.
Same public functions as the reference's ``utils/sft_messages.py:1-199``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Iterable


@dataclass(frozen=True)
class EncodedSFTExample:
    token_ids: list[int]
    supervised_mask: list[int]


# ------------------------------------------------------------------------------------------------ row -> messages
def _decode_if_json(value: Any) -> Any:
    """Strings that look like a JSON list/object are decoded; anything else is returned unchanged."""
    if isinstance(value, str):
        text = value.strip()
        if text[:1] in ("[", "{"):
            try:
                return json.loads(text)
            except json.JSONDecodeError:
                return value
    return value


def normalize_message_content(content: Any) -> str:
    """Flatten the content field of a message to plain text (multi-part contents keep only their text parts)."""
    if isinstance(content, str):
        return content
    if isinstance(content, dict):
        if isinstance(content.get("text"), str):
            return content["text"]
        raise ValueError(f"unsupported message content mapping: {content!r}")
    if isinstance(content, list):
        pieces = []
        for part in content:
            if isinstance(part, str):
                pieces.append(part)
            elif isinstance(part, dict) and isinstance(part.get("text"), str) and part.get("type") in (None, "text"):
                pieces.append(part["text"])
            elif isinstance(part, dict):
                raise ValueError(f"unsupported non-text message content part: {part!r}")
            else:
                raise ValueError(f"unsupported message content part: {part!r}")
        return "".join(pieces)
    raise ValueError(f"unsupported message content type={type(content)!r}")


def extract_messages(row: dict[str, Any], messages_column: str) -> list[dict[str, str]] | None:
    """The row's transcript with empty turns dropped, or None when the column is absent / not a list / all empty."""
    if messages_column not in row:
        return None
    raw = _decode_if_json(row.get(messages_column))
    if not isinstance(raw, list):
        return None
    turns: list[dict[str, str]] = []
    for item in raw:
        if not isinstance(item, dict):
            raise ValueError(f"message must be a mapping, got {type(item)!r}")
        role = item.get("role")
        if not (isinstance(role, str) and role):
            raise ValueError(f"message role must be a non-empty string, got {role!r}")
        text = normalize_message_content(item.get("content"))
        if text:
            turns.append({"role": role, "content": text})
    return turns if turns else None


def messages_from_prompt_completion(prompt: Any, completion: Any) -> list[dict[str, str]] | None:
    if isinstance(prompt, str) and isinstance(completion, str) and prompt and completion:
        return [{"role": "user", "content": prompt}, {"role": "assistant", "content": completion}]
    return None


def has_supervised_assistant_turn(messages: Iterable[dict[str, str]]) -> bool:
    return any(m["role"] == "assistant" and m["content"] for m in messages)


# ------------------------------------------------------------------------------------------------ messages -> tokens
def encode_messages_with_chat_template(messages: list[dict[str, str]], *, tokenizer, assistant_only_loss: bool) -> EncodedSFTExample:
    if not getattr(tokenizer, "chat_template", None):
        raise ValueError("tokenizer does not define a chat_template; rerun with --no-apply-chat-template or choose a chat tokenizer")
    enc = tokenizer.apply_chat_template(messages, tokenize=True, add_generation_prompt=False, return_dict=True,
                                        return_assistant_tokens_mask=assistant_only_loss)
    ids = [int(t) for t in enc["input_ids"]]
    if not assistant_only_loss:
        return EncodedSFTExample(ids, [1] * len(ids))
    masks = enc.get("assistant_masks")
    if masks is None:
        raise ValueError("chat template did not return assistant_masks; the tokenizer template likely needs {% generation %} support")
    mask = [int(m) for m in masks]
    if mask and not any(mask):
        raise ValueError("chat template returned assistant_masks but all values are 0; the tokenizer template likely needs "
                         "{% generation %} blocks around assistant content")
    return EncodedSFTExample(ids, mask)


def encode_messages_plain(messages: list[dict[str, str]], *, tokenizer, assistant_only_loss: bool, append_eos: bool) -> EncodedSFTExample:
    """Template-free rendering: every turn becomes ``"<role>: " + content (+ eos)``. With assistant-only loss the
    supervised tokens are the content and eos of assistant turns (not the role prefix)."""
    eos = tokenizer.eos_token_id
    tail = [int(eos)] if (append_eos and eos is not None) else []
    ids: list[int] = []
    mask: list[int] = []
    for turn in messages:
        head = [int(t) for t in tokenizer.encode(f"{turn['role']}: ", add_special_tokens=False)]
        body = [int(t) for t in tokenizer.encode(turn["content"], add_special_tokens=False)]
        ids += head + body + tail
        if not assistant_only_loss:
            mask += [1] * (len(head) + len(body) + len(tail))
        elif turn["role"] == "assistant":
            mask += [0] * len(head) + [1] * (len(body) + len(tail))
        else:
            mask += [0] * (len(head) + len(body) + len(tail))
    return EncodedSFTExample(ids, mask)


def encode_sft_example(row: dict[str, Any], *, tokenizer, messages_column: str, prompt_column: str, completion_column: str,
                       apply_chat_template: bool, assistant_only_loss: bool, append_eos: bool) -> EncodedSFTExample | None:
    """None when the row has neither a usable transcript nor a prompt/completion pair, or (with assistant-only loss)
    when no assistant turn would be supervised."""
    messages = extract_messages(row, messages_column)
    if messages is None:
        messages = messages_from_prompt_completion(row.get(prompt_column), row.get(completion_column))
    if messages is None:
        return None
    if assistant_only_loss and not has_supervised_assistant_turn(messages):
        return None
    if apply_chat_template:
        return encode_messages_with_chat_template(messages, tokenizer=tokenizer, assistant_only_loss=assistant_only_loss)
    return encode_messages_plain(messages, tokenizer=tokenizer, assistant_only_loss=assistant_only_loss, append_eos=append_eos)
