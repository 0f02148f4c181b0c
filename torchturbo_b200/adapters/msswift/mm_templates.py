"""ms-swift multimodal templates for the vision-language families of this package (Bailing-VL, Kimi-K2.5).

A swift `Template` turns one sample into token ids; for a medium it asks `replace_tag(media_type, index, inputs)`
for the text that stands for it.  The templates here run the family's own image / video processor on that one medium,
expand its tag to as many placeholder tokens as the model will get features for, and hand the processed tensors to the
batch (`pixel_values` + `image_grid_thw`, or `grid_thws` for Kimi); `_data_collator_mm_data` joins the media of the
samples of a batch.  The fusion of features and token embeddings happens inside the models (`fuse_media`), which also
keep their tower in the autograd graph on media-less batches, so there is no `_post_encode` step.

Counts per medium:
  * Bailing-VL (Qwen-VL tower): `t * h * w / merge^2` tokens between `vision_start` and `vision_end`;
  * Kimi-K2.5 (MoonViT, frames pooled): `h * w / merge^2` pad tokens inside
    `<|media_begin|>image<|media_content|> ... <|media_end|>`; a clip is a sequence of such chunks, each behind its
    time stamp.
The classes are built against the `Template` base that is passed in, so they can be built against swift's or a
stand-in's (models/bailing_moe_v3_vl/swift_template.py:145-316 of the reference is the Bailing counterpart; the reference
has no swift template for Kimi-K2.5, only a LlamaFactory plugin)."""
from __future__ import annotations

from typing import Any, Sequence

from ..mm_tokens import kimi_image_piece, kimi_video_piece, tokens_per_grid

_KEY = "tt_media_inputs"


def _rows(grid) -> list[list[int]]:
    return grid.tolist() if hasattr(grid, "tolist") else [list(g) for g in grid]


def join_media(media: Sequence[dict[str, Any]]) -> dict[str, Any]:
    """Media tensors of several media / samples -> one batch entry per key (rows concatenated on dim 0)."""
    import torch

    out: dict[str, Any] = {}
    for key in ("pixel_values", "image_grid_thw", "pixel_values_videos", "video_grid_thw", "grid_thws"):
        parts = [m[key] for m in media if m.get(key) is not None]
        if parts:
            out[key] = torch.cat([torch.as_tensor(p) for p in parts], dim=0)
    return out


def make_swift_mm_templates(base: type) -> dict[str, type]:
    class _MediaTemplate(base):  # type: ignore[misc, valid-type]
        support_padding_free = True

        def _encode(self, inputs):
            inputs.mm_processor_kwargs[_KEY] = []
            encoded = super()._encode(inputs)
            encoded.update(join_media(inputs.mm_processor_kwargs.pop(_KEY)))
            return encoded

        def _data_collator_mm_data(self, batch):
            return join_media(batch)

        def _note(self, inputs, media_inputs) -> None:
            inputs.mm_processor_kwargs.setdefault(_KEY, []).append(dict(media_inputs))

    class BailingVLTemplate(_MediaTemplate):
        """`<image>` -> vision_start + image_token x n + vision_end with n from the processed grid."""

        def replace_tag(self, media_type, index, inputs):
            proc = self.processor
            ip = proc.image_processor
            if media_type == "image":
                media = ip(images=[inputs.images[index]], return_tensors="pt")
                n = tokens_per_grid(_rows(media["image_grid_thw"]), ip.merge_size)[0]
                text = proc.vision_start_token + proc.image_token * n + proc.vision_end_token
            elif media_type == "video":
                vp = getattr(proc, "video_processor", ip)
                media = vp(videos=[inputs.videos[index]], return_tensors="pt")
                n = tokens_per_grid(_rows(media["video_grid_thw"]), ip.merge_size)[0]
                start = getattr(proc, "video_start_token", proc.vision_start_token)
                end = getattr(proc, "video_end_token", proc.vision_end_token)
                text = start + proc.video_token * n + end
            else:
                raise ValueError("Bailing-VL takes images and videos only")
            self._note(inputs, media)
            return [text]

    class KimiK25Template(_MediaTemplate):
        """`<image>` / `<video>` -> Kimi's media pieces with the pad-token counts of the checkpoint's media processor."""

        pad = "<|media_pad|>"

        def replace_tag(self, media_type, index, inputs):
            mp = self.processor.media_processor
            merge = int(getattr(mp, "merge_size", 2))
            if media_type == "image":
                media = mp(images=[inputs.images[index]], return_tensors="pt")
                t, h, w = _rows(media["grid_thws"])[0]
                text = kimi_image_piece(int(h) * int(w) // (merge * merge), self.pad)
            elif media_type == "video":
                chunks = mp.split_video_chunks(inputs.videos[index])          # [(time stamp, frames), ...]
                media = mp(images=[c[1] for c in chunks], return_tensors="pt")
                counts = [int(h) * int(w) // (merge * merge) for _, h, w in _rows(media["grid_thws"])]
                text = kimi_video_piece([(c[0], n) for c, n in zip(chunks, counts)], self.pad)
            else:
                raise ValueError("Kimi-K2.5 takes images and videos only")
            self._note(inputs, media)
            return [text]

    return {"bailing_vl": BailingVLTemplate, "kimi_k25": KimiK25Template}


def register_swift_mm_templates(names: Sequence[str] = ("bailing_vl", "kimi_k25")) -> list[str]:
    """Register the `turbo_bailing_vl` / `turbo_kimi_k25_vl` templates: the chat format of the family (`adapters/chat_templates.py`) with the
    media-aware template class.  Needs ms-swift; returns the registered template names."""
    from copy import copy

    from swift.template import Template, register_template
    from swift.template.register import TEMPLATE_MAPPING

    from ..chat_templates import register_swift_templates

    chat_of = {"bailing_vl": "bailing_v3", "kimi_k25": "kimi_k25"}
    classes = make_swift_mm_templates(Template)
    done = []
    for name in names:
        text_name = register_swift_templates([chat_of[name]])[0]
        meta = copy(TEMPLATE_MAPPING[text_name])
        meta.template_type = f"turbo_{name}" if name.endswith("_vl") else f"turbo_{name}_vl"
        meta.template_cls = classes[name]
        try:
            register_template(meta, exist_ok=True)
        except TypeError:
            register_template(meta)
        done.append(meta.template_type)
    return done
