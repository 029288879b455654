"""Synthetic image + text samples (no dataset download): a 720x480 RGB image and ``"<image>" + " text" * 256``
(the sample shape of the reference's examples/fake_dataset.py)."""

import torch
from torch.utils.data import Dataset


class FakeVisionDataset(Dataset):
    def __init__(self, n: int = 64, height: int = 480, width: int = 720, words: int = 256, seed: int = 0):
        self.n, self.h, self.w, self.words, self.seed = n, height, width, words, seed

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed + i)
        return {"image": torch.rand(3, self.h, self.w, generator=g), "text": "<image>" + " text" * self.words}


def collate(samples, image_size: int):
    images = torch.stack([torch.nn.functional.interpolate(s["image"][None], size=(image_size, image_size))[0] for s in samples])
    return {"pixel_values": images, "text": [s["text"] for s in samples]}
