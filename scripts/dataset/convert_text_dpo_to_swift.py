"""Plain-text preference pairs `{"prompt", "chosen", "rejected"}` -> ms-swift DPO JSON lines."""
from __future__ import annotations

import json
import sys


def convert_record(r: dict) -> dict:
    return {"messages": [{"role": "user", "content": r["prompt"]}, {"role": "assistant", "content": r["chosen"]}],
            "rejected_response": r["rejected"]}


def main(argv=None):
    src, dst = (sys.argv[1:] if argv is None else argv)[:2]
    rows = [json.loads(l) for l in open(src) if l.strip()]
    with open(dst, "w") as f:
        for r in rows:
            f.write(json.dumps(convert_record(r), ensure_ascii=False) + "\n")
    return len(rows)


if __name__ == "__main__":
    main()
