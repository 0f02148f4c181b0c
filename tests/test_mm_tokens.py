"""Media placeholder expansion of the adapter layer: pure string functions and the plugin classes built against a
stand-in for LlamaFactory's BasePlugin (fake processors; no framework, no images)."""
import sys
import types

import pytest

from torchturbo_b200.adapters import mm_tokens as M


def test_expand_counts_across_messages():
    msgs = [{"role": "user", "content": "a<image>b<image>"}, {"role": "assistant", "content": "ok"},
            {"role": "user", "content": "<video>c<image>"}, {"role": "user", "content": [{"type": "text"}]}]
    out = M.expand_media_messages(msgs, ["[1]", "[2]", "[3]"], ["[v]"])
    assert [m["content"] for m in out[:3]] == ["a[1]b[2]", "ok", "[v]c[3]"]
    assert out[3]["content"] == [{"type": "text"}]
    assert msgs[0]["content"] == "a<image>b<image>"          # input untouched


def test_expand_mismatch_raises():
    with pytest.raises(ValueError, match="placeholders than images"):
        M.expand_media_messages([{"content": "<image><image>"}], ["x"], [])
    with pytest.raises(ValueError, match="more images than placeholders"):
        M.expand_media_messages([{"content": "<image>"}], ["x", "y"], [])
    assert M.expand_media_messages([{"content": "<image>"}], ["x", "y"], [], strict=False)[0]["content"] == "x"


def test_kimi_pieces():
    assert M.kimi_image_piece(3) == "<|media_begin|>image<|media_content|><|media_pad|><|media_pad|><|media_pad|><|media_end|>"
    stamp = M.kimi_chunk_stamp("00:00:04<|media_begin|>video<|media_content|><|media_pad|><|media_end|>")
    assert stamp == "00:00:04"
    v = M.kimi_video_piece([("00:00:00", 1), ("00:00:04", 2)], pad="P")
    assert v == ("00:00:00<|media_begin|>video<|media_content|>P<|media_end|>"
                 "00:00:04<|media_begin|>video<|media_content|>PP<|media_end|>")


def test_wrap_and_expand_handles_wrapped_and_bare():
    t = M.wrap_and_expand(["x <s><i><e> y <i>", "<i>"], [2, 1, 3], start="<s>", token="<i>", end="<e>")
    assert t == ["x <s><i><i><e> y <s><i><e>", "<s><i><i><i><e>"]
    with pytest.raises(ValueError):
        M.wrap_and_expand(["<i><i>"], [1], start="<s>", token="<i>", end="<e>")


def test_grid_tokens_and_area_cap():
    assert M.tokens_per_grid([[1, 4, 6], [2, 8, 8]], merge_size=2) == [6, 32]
    assert M.cap_area(100, 50, 0) == (100, 50)
    assert M.cap_area(100, 50, 10_000) == (100, 50)
    w, h = M.cap_area(4000, 3000, 1_000_000)
    assert w * h <= 1_000_000 and abs(w / h - 4 / 3) < 0.01 and w * h > 990_000


# ---- plugin classes against a stand-in base -----------------------------------------------------------------------
class _Base:
    expand_mm_tokens = True

    def __init__(self, image_token=None, video_token=None, audio_token=None):
        self.image_token, self.video_token, self.audio_token = image_token, video_token, audio_token

    def _validate_input(self, processor, images, videos, audios):
        assert processor is not None or not (images or videos)

    def _regularize_images(self, images, **kw):
        return {"images": [f"pil:{im}" if isinstance(im, str) else im for im in images]}


class _KimiMedia:
    def get_resize_config(self, item):
        return {"num_tokens": item.get("n", 2) if item["type"] == "video" else len(str(item["image"]))}

    def split_video_chunks(self, video):
        return [{"type": "video", "n": k + 1, "prompt": f"t{k}<|media_begin|>video..."} for k in range(video)]

    def preprocess(self, medias, return_tensors):
        return {"pixel_values": [m["type"] for m in medias], "grid_thws": len(medias), "extra": 1}


def test_kimi_plugin():
    P = M.make_lf_plugins(_Base)["kimi_k25"]
    proc = types.SimpleNamespace(media_processor=_KimiMedia())
    pl = P(image_token="<|media_pad|>", video_token="<|media_pad|>")
    out = pl.process_messages([{"role": "user", "content": "see <image> and <video>!"}], ["abc"], [2], [], proc)
    pad = "<|media_pad|>"
    assert out[0]["content"] == (f"see <|media_begin|>image<|media_content|>{pad * 3}<|media_end|> and "
                                 f"t0<|media_begin|>video<|media_content|>{pad}<|media_end|>"
                                 f"t1<|media_begin|>video<|media_content|>{pad * 2}<|media_end|>!")
    mm = pl.get_mm_inputs(["path.png", 7], [1], [], [2], [1], [], [[0]], proc)
    assert mm == {"pixel_values": ["image", "image", "video"], "grid_thws": 3}


class _Grid(list):
    def tolist(self):
        return [list(g) for g in self]


def _bailing_processor():
    def image_processor(images, return_tensors, do_resize):
        assert do_resize is True
        return {"pixel_values": len(images), "image_grid_thw": _Grid([[1, 4, 4]] * len(images))}
    image_processor.merge_size = 2
    proc = types.SimpleNamespace(
        image_processor=image_processor, image_token="<IMG>", video_token="<VID>", vision_start_token="<vs>",
        vision_end_token="<ve>", video_start_token="<Vs>", video_end_token="<Ve>", image_max_pixels=0, image_min_pixels=0,
        video_inputs=lambda videos: {"video_grid_thw": _Grid([[2, 4, 4]] * len(videos)), "video_timestamps_seconds": [0.0]},
        _expand_video_tokens=lambda texts, media: [t.replace("<VID>", "<VID>" * 8) for t in texts])
    return proc


def test_bailing_plugin_expands_and_wraps():
    P = M.make_lf_plugins(_Base)["bailing_vl"]
    pl, proc = P(), _bailing_processor()
    out = pl.process_messages([{"role": "user", "content": "<image>q<video>"}, {"role": "assistant", "content": "a"}],
                              ["i0"], ["v0"], [], proc)
    assert out[0]["content"] == "<vs>" + "<IMG>" * 4 + "<ve>q<Vs>" + "<VID>" * 8 + "<Ve>"
    assert out[1]["content"] == "a"
    mm = pl.get_mm_inputs(["i0"], ["v0"], [], [1], [1], [], [[0]], proc)
    assert "video_timestamps_seconds" not in mm and mm["pixel_values"] == 1 and "video_grid_thw" in mm
    pl.expand_mm_tokens = False
    out = pl.process_messages([{"role": "user", "content": "<image>"}], ["i0"], [], [], proc)
    assert out[0]["content"] == "<IMG>"


def test_register_with_fake_llamafactory(monkeypatch):
    lf = types.ModuleType("llamafactory")
    data = types.ModuleType("llamafactory.data")
    mm = types.ModuleType("llamafactory.data.mm_plugin")
    extras = types.ModuleType("llamafactory.extras")
    consts = types.ModuleType("llamafactory.extras.constants")
    consts.IMAGE_PLACEHOLDER, consts.VIDEO_PLACEHOLDER = "<image>", "<video>"
    mm.BasePlugin, mm.PLUGINS = _Base, {"qwen2_vl": object}
    mm.register_mm_plugin = lambda name, cls: mm.PLUGINS.__setitem__(name, cls)
    lf.data, data.mm_plugin, lf.extras, extras.constants = data, mm, extras, consts
    for name, mod in (("llamafactory", lf), ("llamafactory.data", data), ("llamafactory.data.mm_plugin", mm),
                      ("llamafactory.extras", extras), ("llamafactory.extras.constants", consts)):
        monkeypatch.setitem(sys.modules, name, mod)
    assert sorted(M.register_lf_mm_plugins()) == ["bailing_vl", "kimi_k25"]
    assert issubclass(mm.PLUGINS["kimi_k25"], _Base)
    assert M.register_lf_mm_plugins() == []                  # second call: nothing new
