"""Media placeholders -> runs of pad tokens, for the vision-language families the adapter frameworks do not know.

The text side of a multimodal sample is plain string work: every `<image>` / `<video>` placeholder of a message
becomes `begin + pad * n + end`, with n the number of vision tokens the model's processor will produce for that
item.  That part lives here as pure functions (testable without any framework); `register_lf_mm_plugins()` wraps
them into LlamaFactory `BasePlugin` subclasses and registers them under the names the chat formats refer to
(`ChatFormat.mm_plugin`).  Same job as models/kimi_k25/mm_plugin.py:38-138 and
models/bailing_moe_v3_vl/mm_plugin.py:17-141 in the reference; the pixel side is delegated to the checkpoint's own
processor in both.
"""
from __future__ import annotations

import math
import re
from copy import deepcopy
from typing import Any, Callable, Iterable, Iterator, Sequence

from ..logging import get_logger

logger = get_logger(__name__)

IMAGE_PLACEHOLDER = "<image>"
VIDEO_PLACEHOLDER = "<video>"


# ---- pure string work -----------------------------------------------------------------------------------------------
def _substitute(text: str, placeholder: str, pieces: Iterator[str], what: str) -> str:
    """Replace each occurrence of `placeholder`, left to right, by the next item of `pieces`."""
    parts = text.split(placeholder)
    out = [parts[0]]
    for tail in parts[1:]:
        try:
            out.append(next(pieces))
        except StopIteration:
            raise ValueError(f"more {placeholder} placeholders than {what} in the sample") from None
        out.append(tail)
    return "".join(out)


def expand_media_messages(messages: Sequence[dict[str, Any]], image_pieces: Iterable[str], video_pieces: Iterable[str],
                          *, strict: bool = True, image_placeholder: str = IMAGE_PLACEHOLDER,
                          video_placeholder: str = VIDEO_PLACEHOLDER) -> list[dict[str, Any]]:
    """Copy of `messages` with the k-th `<image>` replaced by `image_pieces[k]` and the k-th `<video>` by
    `video_pieces[k]`, counted across the whole conversation.  Non-string contents pass through.  With `strict`, left
    over pieces (more media than placeholders) raise as well: a silent mismatch shifts every later image."""
    imgs, vids = iter(image_pieces), iter(video_pieces)
    out = deepcopy(list(messages))
    for m in out:
        c = m.get("content")
        if not isinstance(c, str):
            continue
        if image_placeholder in c:
            c = _substitute(c, image_placeholder, imgs, "images")
        if video_placeholder in c:
            c = _substitute(c, video_placeholder, vids, "videos")
        m["content"] = c
    if strict:
        for it, what in ((imgs, "images"), (vids, "videos")):
            if next(it, None) is not None:
                raise ValueError(f"more {what} than placeholders in the sample")
    return out


def kimi_image_piece(n_tokens: int, pad: str = "<|media_pad|>") -> str:
    return f"<|media_begin|>image<|media_content|>{pad * n_tokens}<|media_end|>"


def kimi_video_piece(chunks: Sequence[tuple[str, int]], pad: str = "<|media_pad|>") -> str:
    """A video is a sequence of chunks, each `timestamp text + begin/video/content + pad * n + end`."""
    return "".join(f"{stamp}<|media_begin|>video<|media_content|>{pad * n}<|media_end|>" for stamp, n in chunks)


def kimi_chunk_stamp(chunk_prompt: str) -> str:
    """The processor's per-chunk prompt starts with the timestamp text; everything before the first
    `<|media_begin|>` is kept."""
    return chunk_prompt.split("<|media_begin|>")[0]


def wrap_and_expand(texts: Sequence[str], counts: Iterable[int], *, start: str, token: str, end: str) -> list[str]:
    """Every bare `token`, and every already wrapped `start token end`, becomes `start + token * n + end` with the
    next count.  Matching the wrapped form first keeps a template that already carries the wrapper from being
    wrapped twice."""
    it = iter(counts)
    pat = re.compile(re.escape(start + token + end) + "|" + re.escape(token))

    def put(_m: re.Match) -> str:
        try:
            n = next(it)
        except StopIteration:
            raise ValueError("more image tokens in the text than image grids") from None
        return start + token * int(n) + end

    return [pat.sub(put, t) for t in texts]


def tokens_per_grid(grid_thw: Iterable[Sequence[int]], merge_size: int) -> list[int]:
    """Vision tokens the language model sees per item: t*h*w patches merged `merge_size` x `merge_size`."""
    return [int(t) * int(h) * int(w) // (merge_size * merge_size) for t, h, w in grid_thw]


def cap_area(width: int, height: int, max_pixels: int) -> tuple[int, int]:
    """Target (width, height) with the aspect ratio kept and the area capped at `max_pixels` (no change when it
    already fits or the cap is off).  Truncating, as the resize in front of the patch alignment does."""
    if max_pixels <= 0 or width * height <= max_pixels:
        return width, height
    ratio = width / height
    h = math.sqrt(max_pixels / ratio)
    return int(h * ratio), int(h)


# ---- LlamaFactory plugin classes -----------------------------------------------------------------------------------
def _as_rows(grid) -> list[list[int]]:
    return grid.tolist() if hasattr(grid, "tolist") else [list(g) for g in grid]


def make_lf_plugins(base: type, image_placeholder: str = IMAGE_PLACEHOLDER, video_placeholder: str = VIDEO_PLACEHOLDER
                    ) -> dict[str, type]:
    """Plugin classes derived from LlamaFactory's `BasePlugin` (passed in, so the classes can be built against a
    stand-in too)."""
    marks = dict(image_placeholder=image_placeholder, video_placeholder=video_placeholder)

    class KimiK25Plugin(base):  # type: ignore[misc, valid-type]
        """Native-resolution images and chunked videos of Kimi K2.5: counts come from the checkpoint's
        `media_processor` (`get_resize_config(item)["num_tokens"]`, `split_video_chunks(video)`)."""

        def process_messages(self, messages, images, videos, audios, processor):
            self._validate_input(processor, images, videos, audios)
            mp = processor.media_processor
            pad = self.image_token or "<|media_pad|>"
            vpad = self.video_token or pad
            img = (kimi_image_piece(mp.get_resize_config({"type": "image", "image": im})["num_tokens"], pad)
                   for im in images)
            vid = (kimi_video_piece([(kimi_chunk_stamp(ch["prompt"]), mp.get_resize_config(ch)["num_tokens"])
                                     for ch in mp.split_video_chunks(v)], vpad) for v in videos)
            return expand_media_messages(messages, img, vid, strict=False, **marks)

        def get_mm_inputs(self, images, videos, audios, imglens, vidlens, audlens, batch_ids, processor):
            self._validate_input(processor, images, videos, audios)
            mp = processor.media_processor
            medias: list[dict[str, Any]] = []
            for im in images:
                if isinstance(im, (str, bytes, dict)) or hasattr(im, "read"):
                    im = self._regularize_images([im])["images"][0]
                medias.append({"type": "image", "image": im})
            for v in videos:
                medias.extend(mp.split_video_chunks(v))
            got = mp.preprocess(medias, return_tensors="pt")
            return {"pixel_values": got["pixel_values"], "grid_thws": got["grid_thws"]}

    class BailingVLPlugin(base):  # type: ignore[misc, valid-type]
        """Ling / Bailing VL: Qwen-style patch grids; images are area-capped before the patch alignment and wrapped
        in the vision start / end tokens; videos go through the processor's own expansion."""

        def _preprocess_image(self, image, image_max_pixels, image_min_pixels, **kwargs):
            image = image.convert("RGB")
            w, h = cap_area(*image.size, image_max_pixels)
            if (w, h) != tuple(image.size):
                image = image.resize((w, h), resample=2)    # 2 = bilinear in PIL
            return image

        def _media(self, images, videos, audios, processor) -> dict[str, Any]:
            self._validate_input(processor, images, videos, audios)
            out: dict[str, Any] = {}
            if images:
                ip = processor.image_processor
                ims = self._regularize_images(images, image_max_pixels=getattr(processor, "image_max_pixels", 0),
                                              image_min_pixels=getattr(processor, "image_min_pixels", 0))["images"]
                align: Callable | None = getattr(processor, "align_image", None)
                if align is not None:
                    ims = [align(im) for im in ims]
                out.update(ip(images=ims, return_tensors="pt", do_resize=align is None))
            if videos:
                out.update(processor.video_inputs(videos) if hasattr(processor, "video_inputs")
                           else processor.video_processor(videos=videos, return_tensors="pt"))
            return out

        def process_messages(self, messages, images, videos, audios, processor):
            self._validate_input(processor, images, videos, audios)
            if hasattr(self, "_validate_messages"):
                self._validate_messages(messages, images, videos, audios)
            vid_piece = processor.video_start_token + processor.video_token + processor.video_end_token
            n_img = sum(m["content"].count(image_placeholder) for m in messages if isinstance(m.get("content"), str))
            n_vid = sum(m["content"].count(video_placeholder) for m in messages if isinstance(m.get("content"), str))
            out = expand_media_messages(messages, [processor.image_token] * n_img, [vid_piece] * n_vid, strict=False,
                                        **marks)
            if not getattr(self, "expand_mm_tokens", True):
                return out
            media = self._media(images, videos, audios, processor)
            texts = [m["content"] for m in out]
            if images:
                counts = tokens_per_grid(_as_rows(media["image_grid_thw"]), processor.image_processor.merge_size)
                texts = wrap_and_expand(texts, counts, start=processor.vision_start_token, token=processor.image_token,
                                        end=processor.vision_end_token)
            if videos:
                texts = processor._expand_video_tokens(texts, media)
            for m, t in zip(out, texts):
                m["content"] = t
            return out

        def get_mm_inputs(self, images, videos, audios, imglens, vidlens, audlens, batch_ids, processor):
            media = self._media(images, videos, audios, processor)
            media.pop("video_timestamps_seconds", None)     # one grid per video; the model expands the time axis
            return media

    return {"kimi_k25": KimiK25Plugin, "bailing_vl": BailingVLPlugin}


def register_lf_mm_plugins() -> list[str]:
    """Register the plugin classes with the installed LlamaFactory.  Returns the names newly registered; an older
    LlamaFactory without a plugin registry gets none (its templates stay text-only)."""
    try:
        from llamafactory.data import mm_plugin as M
    except Exception:  # noqa: BLE001 - not installed
        return []
    try:
        from llamafactory.extras.constants import IMAGE_PLACEHOLDER as IP, VIDEO_PLACEHOLDER as VP
    except Exception:  # noqa: BLE001
        IP, VP = IMAGE_PLACEHOLDER, VIDEO_PLACEHOLDER
    table = getattr(M, "PLUGINS", None)
    reg = getattr(M, "register_mm_plugin", None)
    if not hasattr(M, "BasePlugin") or (table is None and reg is None):
        logger.warning_rank0("this LlamaFactory has no mm plugin registry: multimodal templates stay text-only")
        return []
    done = []
    for name, cls in make_lf_plugins(M.BasePlugin, IP, VP).items():
        if isinstance(table, dict) and name in table:
            continue
        if reg is not None:
            reg(name, cls)
        else:
            table[name] = cls
        done.append(name)
    return done
