"""Pieces shared by the example scripts: a collate function that runs samples through ``MultimodalProcessor`` (the
counterpart of the reference's examples/commons.py:17-33), and stand-ins for a tokenizer and an image processor so that the
examples run without downloading anything.  With real checkpoints, pass a Hugging Face tokenizer / image processor instead:
``MultimodalProcessor`` only needs callables with their interfaces."""

import torch


class WhitespaceTokenizer:
    """Splits on white space, keeps special tokens whole, hashes words into a fixed vocabulary.  Interface subset of a
    Hugging Face tokenizer: ``len``, ``add_special_tokens``, ``convert_tokens_to_ids``, ``__call__`` -> ``input_ids`` +
    ``attention_mask`` (right padded with id 0)."""

    def __init__(self, vocab_size: int, reserved: int = 8):
        self.vocab_size, self.reserved = vocab_size, reserved
        self.special = {"<pad>": 0}

    def __len__(self):
        return self.vocab_size

    def add_special_tokens(self, d):
        for t in d["additional_special_tokens"]:
            if t not in self.special:
                assert len(self.special) <= self.reserved, "more special tokens than reserved ids"
                self.special[t] = self.vocab_size - len(self.special)  # the last ids of the vocabulary
        return len(d["additional_special_tokens"])

    def convert_tokens_to_ids(self, t):
        return self.special[t]

    def __call__(self, text, return_tensors="pt", **kw):
        texts = [text] if isinstance(text, str) else list(text)
        rows = []
        for s in texts:
            for sp in self.special:
                s = s.replace(sp, f" {sp} ")
            rows.append([self.special.get(w, 1 + (hash(w) % (self.vocab_size - self.reserved - 2))) for w in s.split()])
        n = max(len(r) for r in rows)
        ids = torch.tensor([r + [0] * (n - len(r)) for r in rows])
        return {"input_ids": ids, "attention_mask": (ids != 0).long()}


class ResizeImageProcessor:
    """Resizes to a square and normalises to zero mean / unit variance per image: the job of a Hugging Face image
    processor, on tensors."""

    def __init__(self, size: int):
        self.size = size

    def __call__(self, images=None, return_tensors="pt"):
        out = []
        for im in images:
            im = torch.nn.functional.interpolate(im[None].float(), size=(self.size, self.size), mode="bilinear", align_corners=False)[0]
            out.append((im - im.mean()) / (im.std() + 1e-6))
        return {"pixel_values": torch.stack(out)}


def collate_fn(samples: list[dict], processor, dtype=torch.float32) -> dict:
    """``samples``: dicts with ``"image"`` (a ``[3, H, W]`` tensor) and ``"text"`` (containing the image token once).
    Returns what ``MultimodalModel.forward`` takes; the labels equal the input ids (the model ignores the positions of
    modality tokens and shifts the rest)."""
    batch = processor(encoder_inputs={"vision": {"images": [s["image"] for s in samples]}},
                      llm_inputs={"text": [s["text"] for s in samples], "padding": True}, return_tensors="pt")
    out = {k: v for k, v in batch.items()}
    out["pixel_values"] = out["pixel_values"].to(dtype)
    labels = out["input_ids"].clone()
    labels[out["attention_mask"] == 0] = -100
    out["labels"] = labels
    out.pop("attention_mask")  # the model builds its bitfield mask from the token ids; padding is id 0 at the end
    return out
