"""ImageNet-100: the ImageFolder subset named by a class list (role of util/datasets.py:5-23, whose list
lives in util/imagenet100.txt; here the list file is given by the user or found next to the data)."""
from __future__ import annotations

from pathlib import Path
from typing import Optional

from torchvision.datasets import ImageFolder


class ImageNet100(ImageFolder):
    def __init__(self, root: str, split: str, transform=None, class_list: Optional[str] = None) -> None:
        candidates = [class_list, f"{root}/imagenet100.txt", str(Path(__file__).with_name("imagenet100.txt"))]
        path = next((c for c in candidates if c and Path(c).exists()), None)
        if path is None:
            raise FileNotFoundError("a class list (one WordNet id per line) is needed for ImageNet-100")
        self._keep = {ln.split()[0] for ln in Path(path).read_text().splitlines() if ln.strip()}
        super().__init__(f"{root}/{split}", transform)

    def find_classes(self, directory: str):
        classes, _ = super().find_classes(directory)
        classes = [c for c in classes if c in self._keep]
        if not classes:
            raise FileNotFoundError(f"none of the listed classes exist under {directory}")
        return classes, {c: i for i, c in enumerate(classes)}
