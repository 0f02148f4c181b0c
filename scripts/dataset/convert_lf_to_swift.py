"""Convert LlamaFactory datasets (alpaca or sharegpt records) to ms-swift `messages` JSON lines.

    python scripts/dataset/convert_lf_to_swift.py in.json out.jsonl [--dpo]
With `--dpo`, records carrying `chosen` / `rejected` become swift preference samples (`rejected_response`)."""
from __future__ import annotations

import json
import sys

_ROLE = {"human": "user", "gpt": "assistant", "system": "system", "user": "user", "assistant": "assistant"}


def convert_record(r: dict, dpo: bool = False) -> dict:
    msgs = []
    if r.get("system"):
        msgs.append({"role": "system", "content": r["system"]})
    if "conversations" in r:
        msgs += [{"role": _ROLE.get(t.get("from", t.get("role")), "user"), "content": t.get("value", t.get("content", ""))}
                 for t in r["conversations"]]
    else:
        prompt = r.get("instruction", "") + ("\n" + r["input"] if r.get("input") else "")
        msgs.append({"role": "user", "content": prompt})
        if not dpo and r.get("output") is not None:
            msgs.append({"role": "assistant", "content": r["output"]})
    out = {"messages": msgs}
    if dpo:
        ch, rj = r["chosen"], r["rejected"]
        text = lambda x: x.get("value", x.get("content")) if isinstance(x, dict) else x  # noqa: E731
        out["messages"].append({"role": "assistant", "content": text(ch)})
        out["rejected_response"] = text(rj)
    if r.get("images"):
        out["images"] = r["images"]
    return out


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    dpo = "--dpo" in argv
    src, dst = [a for a in argv if not a.startswith("--")][:2]
    data = json.load(open(src)) if src.endswith(".json") else [json.loads(l) for l in open(src) if l.strip()]
    with open(dst, "w") as f:
        for r in data:
            f.write(json.dumps(convert_record(r, dpo), ensure_ascii=False) + "\n")
    return len(data)


if __name__ == "__main__":
    main()
