"""TEST INFRASTRUCTURE ONLY: plain-Python restatement of wgml's tokenizers and default chat template, the checker
the C++ implementations are compared with.  Nothing in the product imports this file.

Follows crates/wgml/src/models/llama2/tokenizer.rs, crates/wgml/src/models/gpt2/tokenizer.rs and
crates/wgml-chat/src/chat_template.rs + crates/wgml/src/models/llama2/llama-2-chat.jinja line by line.
Parity unpinned: the reference holds no test or fixture for any of them (no vocabulary is in the tree); the
rendering of the chat template additionally restates minijinja's documented white-space rules
(`trim_blocks`: the first newline after a block tag is removed; `lstrip_blocks` off) rather than running it."""
from __future__ import annotations

import regex


class LlamaTokenizer:
    def __init__(self, vocab, scores, bos, eos, unk):
        self.vocab, self.scores, self.bos, self.eos, self.unk = list(vocab), list(scores), bos, eos, unk
        self.index = {}
        for n, v in enumerate(self.vocab):      # tokenizer.rs:38-41
            self.index[v] = n

    def encode(self, text: str, bos: bool, eos: bool):   # tokenizer.rs:75-164
        text = text.replace(" ", "▁")
        tokens = [self.bos] if bos else []
        for ch in text:
            if ch in self.index:
                tokens.append(self.index[ch])
            else:
                tokens.extend(b + 3 for b in ch.encode("utf-8"))
        i = 0
        while i < max(len(tokens) - 2, 0):
            if self.vocab[tokens[i]] + self.vocab[tokens[i + 1]] + self.vocab[tokens[i + 2]] == "<s>":
                tokens[i] = self.bos
                del tokens[i + 2]
                del tokens[i + 1]
            i += 1
        i = 0
        while i < max(len(tokens) - 3, 0):
            if "".join(self.vocab[t] for t in tokens[i:i + 4]) == "</s>":
                tokens[i] = self.eos
                del tokens[i + 3]
                del tokens[i + 2]
                del tokens[i + 1]
            i += 1
        while True:
            best_score, best_id, best_idx = float("-inf"), 0, None
            for i in range(len(tokens) - 1):
                pair = self.vocab[tokens[i]] + self.vocab[tokens[i + 1]]
                if pair in self.index and self.scores[self.index[pair]] > best_score:
                    best_score, best_id, best_idx = self.scores[self.index[pair]], self.index[pair], i
            if best_idx is None:
                break
            tokens[best_idx] = best_id
            del tokens[best_idx + 1]
        if eos:
            tokens.append(self.eos)
        return tokens

    def decode(self, prev_token: int, token: int) -> str:   # tokenizer.rs:166-177
        piece = self.vocab[token]
        if prev_token == 1:
            piece = piece.lstrip()
        if piece.startswith("<0x"):
            try:
                return chr(int(piece[3:5], 16))
            except ValueError:
                pass
        return piece.replace("▁", " ")


def bytes_to_unicode():   # gpt2/tokenizer.rs:22-36
    bs = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


class Gpt2Tokenizer:
    PAT = regex.compile(r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+")   # tokenizer.rs:75
    SPECIAL = regex.compile(r"<[^<>]*>")                                                          # tokenizer.rs:128

    def __init__(self, vocab, merges, bos, eos):
        self.bos, self.eos = bos, eos
        self.vocab = list(vocab)
        self.encoder = {s: i for i, s in enumerate(self.vocab)}
        self.merges = {}
        for i, line in enumerate(merges):
            a, b = line.split()[:2]
            self.merges[(a, b)] = i
        self.byte_encoder = bytes_to_unicode()
        self.byte_decoder = {c: b for b, c in self.byte_encoder.items()}

    def bpe(self, token: str):   # tokenizer.rs:170-216
        word = list(token)
        if len(word) < 2:
            return word
        while True:
            pairs = {(word[i], word[i + 1]) for i in range(len(word) - 1)}
            first, second = min(pairs, key=lambda p: (self.merges.get(p, float("inf")),))
            if (first, second) not in self.merges:
                break
            new, i = [], 0
            while i < len(word):
                if first in word[i:]:
                    j = word[i:].index(first)
                    new.extend(word[i:i + j])
                    i += j
                    if i < len(word) - 1 and word[i + 1] == second:
                        new.append(first + second)
                        i += 2
                    else:
                        new.append(word[i])
                        i += 1
                else:
                    new.extend(word[i:])
                    break
            word = new
            if len(word) == 1:
                break
        return word

    def _tokenize(self, sub: str, out):
        for m in self.PAT.finditer(sub):
            enc = "".join(self.byte_encoder[b] for b in m.group().encode("utf-8"))
            for sym in self.bpe(enc):
                if sym in self.encoder:
                    out.append(self.encoder[sym])

    def encode(self, text: str):   # tokenizer.rs:108-146
        out, cursor = [], 0
        for m in self.SPECIAL.finditer(text):
            if cursor != m.start():
                self._tokenize(text[cursor:m.start()], out)
            out.append(self.encoder[m.group()])
            cursor = m.end()
        if cursor < len(text):
            self._tokenize(text[cursor:], out)
        return out

    def decode(self, tokens) -> str:   # tokenizer.rs:156-168
        text = "".join(self.vocab[t] for t in tokens if 0 <= t < len(self.vocab))
        return "".join(chr(self.byte_decoder[c]) for c in text if c in self.byte_decoder)


def chat_template_llama2(messages, bos: str, eos: str) -> str:
    """llama-2-chat.jinja under minijinja with trim_blocks (chat_template.rs:27-39).  The literal text of the
    template between its tags (indentation, blank lines) is emitted exactly as written there, minus the one
    newline trim_blocks removes after each `{% ... %}`."""
    out = []
    if messages[0][0] == "system":
        out.append("    ")      # indentation of `{% set system_message ... %}`
        system_message = "<<SYS>>\n" + messages[0][1].strip() + "\n<</SYS>>\n\n"
        out.append("    ")      # indentation of `{% set messages = messages[1:] %}`
        messages = messages[1:]
    else:
        out.append("    ")      # indentation of `{% set system_message = '' %}`
        system_message = ""
    out.append("\n")            # the blank line after `{% endif %}`
    for index0, (role, content) in enumerate(messages):
        out.append("    ")      # indentation of the alternation check
        if (role == "user") != (index0 % 2 == 0):
            raise ValueError("Conversation roles must alternate user/assistant/user/assistant/...")
        out.append("\n")        # blank line after its `{% endif %}`
        out.append("    ")      # indentation of `{% if loop.index0 == 0 %}`
        out.append("        ")  # indentation of the `{% set content ... %}` of the branch taken
        content = system_message + content if index0 == 0 else content
        out.append("    ")      # indentation of the `{% else %}` / `{% endif %}` that ends the branch
        out.append("\n")        # blank line
        out.append("    ")      # indentation of `{% if message['role'] == 'user' %}`
        if role == "user":
            out.append("        " + bos + "[INST] " + content.strip() + " [/INST]" + "\n")
            out.append("    ")  # indentation of `{% elif ... %}`
        elif role == "assistant":
            out.append("        " + " " + content.strip() + " " + eos + "\n")
            out.append("    ")  # indentation of `{% endif %}`
    return "".join(out)
