"""ms-swift multimodal templates (Bailing-VL, Kimi-K2.5) against a stand-in `Template` base and stand-in processors:
tag expansion with the right number of placeholder tokens, media tensors carried into the encoded sample and joined
across a batch, registration."""
import sys
import types

import pytest
import torch

from torchturbo_b200.adapters.msswift import mm_templates as MT


class _Inputs:
    def __init__(self, text, images=(), videos=()):
        self.text, self.images, self.videos = text, list(images), list(videos)
        self.mm_processor_kwargs = {}


class _BaseTemplate:
    """What the tests need of swift's `Template`: `_encode` walks the text and asks `replace_tag` per media tag."""

    def __init__(self, processor):
        self.processor = processor

    def _encode(self, inputs):
        out, counts = [], {"image": 0, "video": 0}
        for piece in inputs.text.replace("<image>", "\0image\0").replace("<video>", "\0video\0").split("\0"):
            if piece in counts:
                out += self.replace_tag(piece, counts[piece], inputs)
                counts[piece] += 1
            elif piece:
                out.append(piece)
        return {"text": "".join(out)}


class _ImageProcessor:
    merge_size = 2

    def __call__(self, images=None, videos=None, return_tensors=None):
        items = images if images is not None else videos
        if videos is not None:
            grid = torch.tensor([[f, h, w] for f, h, w in items])
            return {"pixel_values_videos": torch.ones(int(grid.prod(-1).sum()), 6), "video_grid_thw": grid}
        grid = torch.tensor([[1, h, w] for h, w in items])
        return {"pixel_values": torch.ones(int(grid.prod(-1).sum()), 6), "image_grid_thw": grid}


class _BailingProcessor:
    image_processor = _ImageProcessor()
    vision_start_token, vision_end_token, image_token, video_token = "<S>", "<E>", "<I>", "<V>"


class _KimiMedia:
    merge_size = 2

    def __call__(self, images=None, return_tensors=None):
        grid = torch.tensor([[1, h, w] for h, w in images])
        return {"pixel_values": torch.ones(int(grid.prod(-1).sum()), 3, 14, 14), "grid_thws": grid}

    def split_video_chunks(self, video):
        return [(stamp, frame) for stamp, frame in video]


class _KimiProcessor:
    media_processor = _KimiMedia()


def test_bailing_vl_expands_tags_and_carries_media():
    T = MT.make_swift_mm_templates(_BaseTemplate)["bailing_vl"](_BailingProcessor())
    enc = T._encode(_Inputs("a<image>b<video>c<image>", images=[(4, 4), (2, 6)], videos=[(2, 4, 4)]))
    assert enc["text"] == "a<S>" + "<I>" * 4 + "<E>b<S>" + "<V>" * 8 + "<E>c<S>" + "<I>" * 3 + "<E>"
    assert enc["image_grid_thw"].tolist() == [[1, 4, 4], [1, 2, 6]] and enc["pixel_values"].shape == (28, 6)
    assert enc["video_grid_thw"].tolist() == [[2, 4, 4]] and enc["pixel_values_videos"].shape == (32, 6)
    with pytest.raises(ValueError):
        T.replace_tag("audio", 0, _Inputs(""))
    batch = T._data_collator_mm_data([enc, T._encode(_Inputs("<image>", images=[(2, 2)])), {"text": "no media"}])
    assert batch["image_grid_thw"].tolist() == [[1, 4, 4], [1, 2, 6], [1, 2, 2]] and batch["pixel_values"].shape[0] == 32


def test_kimi_k25_pieces_pool_frames():
    T = MT.make_swift_mm_templates(_BaseTemplate)["kimi_k25"](_KimiProcessor())
    enc = T._encode(_Inputs("x<image>y<video>", images=[(4, 6)], videos=[[("00:00:00", (2, 2)), ("00:00:04", (4, 4))]]))
    pad = "<|media_pad|>"
    assert enc["text"].startswith("x<|media_begin|>image<|media_content|>" + pad * 6 + "<|media_end|>y")
    assert enc["text"].count(pad) == 6 + 1 + 4 and "00:00:04" in enc["text"]
    assert enc["grid_thws"].tolist() == [[1, 4, 6], [1, 2, 2], [1, 4, 4]] and enc["pixel_values"].shape == (44, 3, 14, 14)


def test_registration_builds_on_the_family_chat_format(monkeypatch):
    mapping = {}

    class TemplateMeta:
        def __init__(self, template_type, **kw):
            self.template_type, self.template_cls = template_type, None
            self.__dict__.update(kw)

    def register_template(meta, exist_ok=False):
        mapping[meta.template_type] = meta

    mods = {"swift": {}, "swift.template": {"register_template": register_template, "Template": _BaseTemplate},
            "swift.template.template_meta": {"TemplateMeta": TemplateMeta},
            "swift.template.register": {"TEMPLATE_MAPPING": mapping, "register_template": register_template}}
    for name, attrs in mods.items():
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        monkeypatch.setitem(sys.modules, name, m)
    done = MT.register_swift_mm_templates()
    assert done == ["turbo_bailing_vl", "turbo_kimi_k25_vl"]
    assert issubclass(mapping["turbo_kimi_k25_vl"].template_cls, _BaseTemplate)
    assert mapping["turbo_bailing_v3"].template_cls is None          # the text format stays registered on its own
    assert mapping["turbo_bailing_vl"].prompt == mapping["turbo_bailing_v3"].prompt
