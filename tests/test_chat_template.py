"""The chat template against literal strings written from the reference's
function (crane/src/llm/client.rs:299-336, hunyuan_dense/model.rs:178-190)."""
from crane_b200.generation import apply_chat_template, format_chat

BAR, LOW = "｜", "▁"
BOS = f"<{BAR}hy_begin{LOW}of{LOW}sentence{BAR}>"
USER = f"<{BAR}hy_User{BAR}>"
ASSISTANT = f"<{BAR}hy_Assistant{BAR}>"
EOS = f"<{BAR}hy_place{LOW}holder{LOW}no{LOW}2{BAR}>"
SEP = f"<{BAR}hy_place{LOW}holder{LOW}no{LOW}3{BAR}>"


def test_one_user_message():
    assert format_chat("hi there") == BOS + USER + "hi there" + ASSISTANT
    assert apply_chat_template([{"role": "user", "content": "hi there"}]) == BOS + USER + "hi there" + ASSISTANT


def test_system_message_and_turns():
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "a"},
            {"role": "assistant", "content": "b"}, {"role": "tool", "content": "dropped"},
            {"role": "user", "content": "c"}]
    assert apply_chat_template(msgs) == (BOS + "be brief" + SEP + USER + "a" + ASSISTANT + "b" + EOS
                                         + USER + "c" + ASSISTANT)
    assert format_chat("q", system="s") == BOS + "s" + SEP + USER + "q" + ASSISTANT


def test_a_system_message_counts_only_in_first_place():
    msgs = [{"role": "user", "content": "a"}, {"role": "system", "content": "late"}]
    assert apply_chat_template(msgs) == BOS + USER + "a" + ASSISTANT
    assert apply_chat_template([]) == BOS + ASSISTANT
