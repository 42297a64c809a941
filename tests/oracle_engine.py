"""Test infrastructure: the Engine interface implemented with the CPU oracle, so
that the scheduler can be run end to end against it and its output compared
with the CUDA engine's."""
import numpy as np
import torch

from oracle import oracle
from whisperdrz_b200.rules import timestamp_tables


def rule_from_words(w) -> dict:
    w = [int(v) for v in w]
    if w[0] >= 0:
        return {"forced_id": w[0]}
    return {"mode": w[1], "arg0": w[2], "arg1": w[3], "table_bits": w[4] & 0xFFFFFFFF, "prefix_begin": w[5],
            "prefix_end": w[6], "set_ids": w[8: 8 + w[7]], "or_table": w[14], "allow_table": w[15], "clear_ids": w[17: 17 + w[16]],
            "pen_ids": w[22: 22 + w[21]]}


class OracleEngine:
    device = torch.device("cpu")

    def __init__(self, dims, sd, n_slots, max_clips=16):
        self.dims, self.sd = dims, sd
        self.n_slots, self.max_clips, self.max_tokens = n_slots, max_clips, dims.n_text_ctx
        self.dec = oracle.SlotDecoder(sd, dims.n_text_layer, dims.n_text_head, n_slots, dims.n_text_ctx)
        self.tables = timestamp_tables(dims.n_vocab)

    def device_status(self):
        pass

    def logmel(self, buf, n_samples=None, frame_offset=None):
        out = []
        for i in range(buf.shape[0]):
            n = buf.shape[1] if n_samples is None else int(n_samples[i])
            off = 0 if frame_offset is None else int(frame_offset[i])
            out.append(oracle.window_mel(oracle.log_mel(buf[i, :n].clone()), off))
        return torch.stack(out)

    def encode(self, mel):
        return oracle.encoder(self.sd, mel, self.dims.n_audio_layer, self.dims.n_audio_head)

    def prefill(self, xa, slots, prompts):
        return self.dec.prefill(torch.tensor(prompts), xa, [int(s) for s in slots])[:, -1]

    def _rules(self, rules, n):
        if rules is None:
            return [{} for _ in range(n)]
        return [rule_from_words(r) for r in np.asarray(rules)]

    def rules_argmax(self, logits, rules):
        return oracle.rules_argmax(logits, self._rules(rules, logits.shape[0]), self.tables).to(torch.int32)

    def decode_step(self, tokens, slots, rules=None):
        logits = torch.cat([self.dec.forward(torch.tensor([[int(t)]]), [int(s)])[:, 0] for t, s in zip(tokens, slots)])
        return self.rules_argmax(logits, rules)
