"""Host-side feeder for embedding inference: token-id lists in, pooled embeddings out.

Mirrors what the reference's `M2_BERT_Encoder.encode_queries / encode_corpus` do around the model
(bert/embeddings_inference.py:267-351): every text is padded (or cut) to ONE evaluation length -- the
mixer convolves padded positions like any other, so the padded length is part of the function being
computed and length bucketing would change the embeddings -- the attention mask marks the real tokens,
the model's pooled output is collected on the host as float32 and checked for NaNs.  What differs is
the plumbing: the reference tokenises and concatenates one text at a time on the device; here a chunk
is assembled in pinned host memory, sent with one copy and run through one CUDA-graph replay per chunk
(the last, shorter chunk is padded with empty rows and cropped).  Tokenisation stays with the caller:
no tokenizer files ship with this package.
"""
from __future__ import annotations

import numpy as np
import torch

from .graph import GraphedForward


class M2BertEmbedder:
    """embedder = M2BertEmbedder(model, max_len, batch_size); vectors = embedder.encode(list_of_id_lists).

    model: an `m2_b200.encoder.M2BertModel` built with `add_pooling_layer=True`, on a CUDA device, in
    eval mode.  encode() returns a float32 numpy array (n_texts, hidden_size).
    """

    def __init__(self, model, max_len, batch_size, pad_token_id=None, use_graph=True):
        if model.pooler is None:
            raise ValueError("M2BertEmbedder needs a model built with add_pooling_layer=True")
        self.model = model.eval()
        self.max_len, self.batch_size = int(max_len), int(batch_size)
        self.pad = model.config.pad_token_id if pad_token_id is None else int(pad_token_id)
        self.device = next(model.parameters()).device
        pin = self.device.type == "cuda"
        self._ids = torch.empty((self.batch_size, self.max_len), dtype=torch.long, pin_memory=pin)
        self._mask = torch.empty((self.batch_size, self.max_len), dtype=torch.long, pin_memory=pin)
        self._graphed = None
        self.use_graph = bool(use_graph) and pin

    def _fill(self, chunk):
        """Pad / cut the chunk's id lists into the pinned staging tensors; rows past the chunk are empty."""
        self._ids.fill_(self.pad)
        self._mask.zero_()
        for i, ids in enumerate(chunk):
            n = min(len(ids), self.max_len)
            self._ids[i, :n] = torch.as_tensor(ids[:n], dtype=torch.long)
            self._mask[i, :n] = 1
        if len(chunk) < self.batch_size:
            self._mask[len(chunk):, 0] = 1              # keeps the mean pooler's denominator non-zero

    def _forward(self, ids, mask):
        out = self.model(ids, attention_mask=mask)
        return out[1]

    def encode(self, token_id_lists):
        out = np.empty((len(token_id_lists), self.model.config.hidden_size), dtype=np.float32)
        for start in range(0, len(token_id_lists), self.batch_size):
            chunk = token_id_lists[start:start + self.batch_size]
            self._fill(chunk)
            if self.use_graph:
                if self._graphed is None:
                    ids, mask = self._ids.to(self.device), self._mask.to(self.device)
                    self._graphed = GraphedForward(self._forward, ids, mask)
                pooled = self._graphed(self._ids, self._mask)
            else:
                with torch.no_grad(), torch.autocast(self.device.type, dtype=torch.bfloat16, enabled=self.device.type == "cuda"):
                    pooled = self._forward(self._ids.to(self.device), self._mask.to(self.device))
            vec = pooled[:len(chunk)].float().cpu().numpy()
            if np.isnan(vec).any():
                raise ValueError("NaNs in the embeddings")      # the reference raises here too
            out[start:start + len(chunk)] = vec
        return out
