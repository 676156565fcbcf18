"""Writes tests/golden/roost_tiny_plain.json: what the plain implementation gives for the reference's roost-tiny.

The reference's own model code is C# and cannot be compiled in an image without a .NET SDK, so these numbers do not
come from running it. They come from tests/plain/qwen3_plain.py on weights made by the reference's seeded generator;
what ties them to the reference are the constants its own tests pin and which the plain implementation reproduces:
the FNV-1a digests of one generated weight slot (tests/Starlings.Roost.Models.Tiny.Tests/TinyWeightsTests.cs:53-54),
the eight greedy token ids of roost-tiny for Prompt(18, 6)
(tests/Starlings.Roost.Models.Tiny.Tests/RoostTinyTests.cs:16,260-293) and three Philox4x32-10 known answers
(tests/Starlings.Roost.Ops.Tests/ElementTests.cs:71-80). Run from the repository root: python tests/golden/make_golden.py
"""
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from tests.plain import qwen3_plain as plain  # noqa: E402


def main():
    cfg, w = plain.roost_tiny_reference_model()
    prompt = [((i * 37) + (6 * 101) + 11) % 256 for i in range(18)]
    logits = plain.forward_logits(cfg, w, prompt)
    out = {
        "reference_pins": {
            "digest_l0_q_proj_f32": 10427801740649689927, "digest_l0_q_proj_bf16": 6253068743922294065,
            "greedy_ids_prompt_18_6": [57, 4, 41, 54, 132, 98, 231, 164],
            "philox": [[[0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]],
                       [[0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]],
                       [[0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0], [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]]],
        },
        "prompt": prompt,
        "plain_greedy": plain.greedy(cfg, w, prompt, 8),
        "plain_last_row_logits": [float(x) for x in logits[-1]],
        "plain_first_row_logits_head": [float(x) for x in logits[0][:16]],
    }
    Path(__file__).with_name("roost_tiny_plain.json").write_text(json.dumps(out, indent=1) + "\n")


if __name__ == "__main__":
    main()
