"""Python restatement of the reference's allocator and step builder.  TEST INFRASTRUCTURE ONLY.

PINNED against the compiled reference (``oracle/_ref``) and the known-answer traces
in ``tests/golden/host_traces.json``.  ``KVStorageRef`` follows
csrc/memory_manager.cpp:4-157; ``BatchSchedulerRef`` follows
csrc/batch_scheduler.h:22-67 and csrc/batch_scheduler.cpp:5-199.  Block-table
padding, which the reference leaves uninitialised, is -1 here; compare only
entries below each request's physical block count.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np


class KVStorageRef:
    def __init__(self, num_blocks: int):
        self.free: List[int] = list(range(num_blocks))          # memory_manager.cpp:4-10
        self.owned: Dict[int, List[int]] = {}
        self.num_allocated = 0
        self.new_allocated = 0

    def allocate(self, size: int) -> np.ndarray:                  # :12-23
        return np.array([self.free.pop() for _ in range(size)], dtype=np.int32)

    def allocate_batch(self, info, L: int, H: int) -> np.ndarray:  # :25-142
        info = np.asarray(info, dtype=np.int64).reshape(-1, 3)
        n = len(info)
        nfree = len(self.free)
        want, need, held = [], [], []
        prefix, run = [], 0
        for rid, nlog, has in info:
            rid = int(rid)
            w = int(nlog) * L * H
            nn = w
            if not has:                                            # :41-48
                if rid in self.owned:
                    nn -= len(self.owned[rid])
                    held.append(len(self.owned[rid]))
                else:
                    held.append(0)
            else:                                                  # :49 (operator[] creates the entry)
                held.append(len(self.owned.setdefault(rid, [])))
            run += nn
            prefix.append(run)
            want.append(w)
            need.append(nn)
        suffix = [0] * (n + 1)
        for i in range(n - 1, -1, -1):                             # :58-62
            suffix[i] = suffix[i + 1] + held[i]
        p = n
        while p >= 0:                                              # :65-72
            if p == 0 or prefix[p - 1] <= nfree + suffix[p]:
                break
            p -= 1
        freed = 0
        for i in range(p, n):                                      # :75-84
            rid = int(info[i][0])
            if held[i] > 0:
                freed += held[i]
                self.free.extend(self.owned.get(rid, []))
                self.owned.pop(rid, None)
        self.num_allocated -= freed                                # :85-86
        self.new_allocated = -freed
        if p <= 0:                                                 # :89-94
            return np.array([p], dtype=np.int32)
        take = prefix[p - 1]
        src = self.free[len(self.free) - take:]                    # :106
        out = [p]
        off = 0
        for i in range(p):                                         # :107-135
            rid = int(info[i][0])
            if need[i] > 0:
                self.owned.setdefault(rid, []).extend(src[off:off + need[i]])
                off += need[i]
            if want[i] > 0:
                out.extend(self.owned[rid][len(self.owned[rid]) - want[i]:])
        self.new_allocated += take                                 # :136-140
        self.num_allocated += self.new_allocated
        del self.free[len(self.free) - take:]
        return np.array(out, dtype=np.int32)

    def free_batch(self, ids) -> int:                              # :144-157
        freed = 0
        for rid in ids:
            rid = int(rid)
            if rid in self.owned:
                freed += len(self.owned[rid])
                self.free.extend(self.owned.pop(rid))
        self.num_allocated -= freed
        return freed

    def get_new_blocks_allocated(self) -> int:
        return self.new_allocated


class _Req:
    def __init__(self, rid, max_tokens, prompt, B, max_blocks, L, H):
        self.id, self.max_tokens, self.B = rid, max_tokens, B
        self.prompt = [int(t) for t in prompt]
        self.outputs: List[int] = []
        self.nphys = 0
        plen = len(self.prompt)
        self.lidx = (plen + B - 1) // B - 1                         # batch_scheduler.h:25-27
        self.loff = (plen - 1) % B
        self.ctx = plen
        self.table = np.full(max_blocks * L * H, -1, dtype=np.int64)


class BatchSchedulerRef:
    def __init__(self, L: int, H: int, max_seq_len: int, B: int):
        self.L, self.H, self.B = L, H, B
        self.max_blocks = (max_seq_len + B - 1) // B                # batch_scheduler.cpp:9
        self.reqs: Dict[int, _Req] = {}
        self.preempted: List[int] = []
        self.prompt_info: List[int] = []
        self.batch_reqs: List[List[int]] = []

    def add_request(self, prompt, rid: int, max_tokens: int) -> None:   # :12-20
        self.reqs[rid] = _Req(rid, max_tokens, prompt, self.B, self.max_blocks, self.L, self.H)

    def try_batch(self, ids, last_tokens) -> np.ndarray:                # :22-48
        decoding = len(last_tokens) > 0
        out, total = [], 0
        for i, rid in enumerate(ids):
            r = self.reqs[int(rid)]
            need = r.lidx + 1
            if decoding:                                                 # batch_scheduler.h:31-40
                r.outputs.append(int(last_tokens[i]))
                r.ctx += 1
                r.loff += 1
                if r.loff == self.B:
                    r.lidx += 1
                    r.loff = 0
                need = r.lidx + 1 - r.nphys
            out += [r.id, need, min(r.nphys, 1)]
            total += need
        return np.array(out + [total], dtype=np.int32)

    def get_batch_info(self, req, block_info) -> List[int]:             # :51-97
        req = np.asarray(req).reshape(-1, 3)
        block_info = np.asarray(block_info)
        LH = self.L * self.H
        p = int(block_info[0])
        off = 1
        ntok = nctx = maxctx = maxblk = 0
        prompts = []
        for i in range(p):
            r = self.reqs[int(req[i][0])]
            need = int(req[i][1]) * LH
            if need > 0:
                r.table[r.nphys * LH:r.nphys * LH + need] = block_info[off:off + need]
                off += need
                r.nphys += int(req[i][1])
            if r.outputs:
                maxblk = max(maxblk, r.nphys)
                maxctx = max(maxctx, r.ctx)
                nctx += 1
                ntok += 1
            else:
                prompts.append(len(r.prompt))
                ntok += len(r.prompt)
        return [ntok, nctx, maxctx, maxblk, self.L, self.H] + prompts

    def get_batch(self, req, block_info, token_tensor, position_tensor, context_len_tensor,
                  block_table_tensor, slot_mapping_tensor) -> None:              # :99-193
        """Fills the caller's CPU tensors like the reference; block-table padding is -1."""
        req = np.asarray(req).reshape(-1, 3)
        LH = self.L * self.H
        p = int(np.asarray(block_info)[0])
        toks, pos, ctxs, slots = [], [], [], []
        self.preempted, self.prompt_info, self.batch_reqs = [], [], []
        maxblk = maxctx = 0
        for i in range(len(req)):
            rid = int(req[i][0])
            if i >= p:                                                   # :123-129
                self.preempted.append(rid)
                self.reqs.pop(rid, None)
                continue
            r = self.reqs[rid]
            if r.outputs:                                                # :132-141
                maxblk = max(maxblk, r.nphys)
                toks.append(r.outputs[-1])
                pos.append(r.ctx - 1)
                ctxs.append(r.ctx)
                maxctx = max(maxctx, r.ctx)
                base = (r.nphys - 1) * LH                                # batch_scheduler.h:58-67
                slots += [int(r.table[base + j]) * self.B + r.loff for j in range(LH)]
            else:                                                        # :142-151, batch_scheduler.h:42-56
                toks += r.prompt
                pos += list(range(len(r.prompt)))
                self.prompt_info.append(len(r.prompt))
                for t in range(len(r.prompt)):
                    base = (t // self.B) * LH
                    slots += [int(r.table[base + j]) * self.B + t % self.B for j in range(LH)]
            self.batch_reqs.append([rid, r.max_tokens])
        self.prompt_info.append(maxctx)
        T = len(toks)
        bt = np.full((T, maxblk, self.L, self.H), -1, dtype=np.int64)
        if maxblk > 0:
            for i in range(p):
                r = self.reqs[int(req[i][0])]
                bt[i].reshape(-1)[:r.nphys * LH] = r.table[:r.nphys * LH]
        tok_np, pos_np = token_tensor.numpy(), position_tensor.numpy()           # :171-192
        tok_np[:T], pos_np[:T] = toks, pos
        tok_np[T:], pos_np[T:] = 0, 0
        context_len_tensor.numpy()[:len(ctxs)] = ctxs
        slot_mapping_tensor.numpy().reshape(-1)[:len(slots)] = slots
        block_table_tensor.numpy().reshape(-1)[:bt.size] = bt.reshape(-1)

    def release_requests(self, ids) -> None:
        for rid in ids:
            self.reqs.pop(int(rid), None)

    def get_preempt_requests(self):
        return list(self.preempted)

    def get_prompt_info(self):
        return list(self.prompt_info)

    def get_batch_reqs(self):
        return [list(x) for x in self.batch_reqs]
