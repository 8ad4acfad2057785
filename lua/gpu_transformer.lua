-- gpu_transformer (B200): the reference's GPU model module with the same constructor, fields and methods
-- (ai/gpu/gpu_transformer.lua:111-887), running on the native device-resident model of luaTL.so instead of
-- queuing per-step op lists from Lua.  Put this directory ahead of ai/gpu on package.path:
--
--   package.path = "lua/?.lua;" .. package.path
--   local GT = require("gpu_transformer")        -- lmtrain_gpu.lua, lmtrain.lua and lmio.lua use it unchanged
--
-- What stays: GT.new{vocab, dim, layers, heads, ffn, max_seq, batch_size, causal, pos, rope_base, tie, dropout,
-- clip_norm, weight_decay, beta1, beta2, graph, timing, want_acc}; fields B, T, N, steps, params[i] = {name, rows,
-- cols, nelem, decay}; train_step -> loss, correct, valid, gnorm, finite; eval_step; forward(ids) -> last-row proxy;
-- capture / maybe_capture; snapshot / restore / release_snapshot; read_param / write_param; free; parameters;
-- nparams; flops_per_step; vram; last_step_ms.  The padding contract is the reference's (:21-27, :567-605).
--
-- What is new: optimizer = "sgd" besides "adamw"; dtype = "bf16"; decode_batch (sequences held by the KV cache);
-- new_state() / step(id, state) / prefill(ids, state) - their presence switches LMTrain:generate onto its cache
-- branch (ai/optim/lmtrain.lua:1499-1519) - and generate_batch(prompts, n_new) for many sequences at once.
--
-- What is gone: params[i].w / .g / .m / .v handles (weights, gradients and optimizer state live in flat device
-- buffers; lmio streams through read_param / write_param as before), and the size threshold / CPU fallback: any
-- non-zero status raises.
local ffi = require("ffi")
local adapter = require("luatl_adapter")

local GT = {}
GT.__index = GT
local Model = {}
Model.__index = Model
GT.Model = Model

local sqrt, floor = math.sqrt, math.floor
local sformat = string.format

local luaTL, lm, C

local function bind()
    if luaTL then return end
    if not adapter.available then
        error("gpu_transformer: luaTL is not available (" .. tostring(adapter.error) .. ").\n" ..
              "  Build the CUDA backend first:  python -m lanternl_b200.build   (nvcc, sm_100a)", 3)
    end
    luaTL = adapter.luaTL
    lm    = require("luaTL_lm")
    C     = luaTL.C
end

local function need(cfg, key)
    local v = cfg[key]
    if type(v) ~= "number" or v ~= floor(v) or v < 1 then
        error(sformat("gpu_transformer: '%s' must be a positive integer, got %s", key, tostring(v)), 3)
    end
    return v
end

function GT.new(cfg)
    bind()
    cfg = cfg or {}
    local self = setmetatable({}, Model)
    self.vocab, self.dim, self.layers = need(cfg, "vocab"), need(cfg, "dim"), need(cfg, "layers")
    self.heads, self.ffn = need(cfg, "heads"), need(cfg, "ffn")
    self.T, self.B = need(cfg, "max_seq"), need(cfg, "batch_size")
    if self.dim % self.heads ~= 0 then
        error(sformat("gpu_transformer: dim (%d) must be divisible by heads (%d)", self.dim, self.heads), 2)
    end
    self.hd = self.dim / self.heads
    if self.hd % 2 ~= 0 then
        error(sformat("gpu_transformer: head_dim (dim/heads = %d) must be even for RoPE", self.hd), 2)
    end
    local pos = string.lower(tostring(cfg.pos or "rope"))
    if pos == "rope" or pos == "rotary" then
        self.use_rope = true
    elseif pos == "none" or pos == "off" then
        self.use_rope = false
    else
        error(sformat("gpu_transformer: pos = '%s' is not supported by the GPU backend.\n" ..
              "  Use pos = 'rope' or pos = 'none', or switch to backend = 'cpu'.", pos), 2)
    end
    if cfg.dropout and cfg.dropout > 0 then
        error(sformat("gpu_transformer: dropout = %g is not supported by the GPU backend", cfg.dropout), 2)
    end
    self.causal       = (cfg.causal ~= false)
    self.tie          = (cfg.tie ~= false)
    self.eps          = cfg.eps or 1e-5
    self.rope_base    = cfg.rope_base or 10000
    self.clip_norm    = cfg.clip_norm or 0
    self.weight_decay = cfg.weight_decay or 0.0
    self.beta1        = cfg.beta1 or 0.9
    self.beta2        = cfg.beta2 or 0.95
    self.adam_eps     = cfg.adam_eps or 1e-8
    self.want_acc     = (cfg.want_acc ~= false)
    self.use_graph    = (cfg.graph == true)
    self.timing       = (cfg.timing == true)
    local opt = string.lower(tostring(cfg.optimizer or "adamw"))
    if opt ~= "adamw" and opt ~= "sgd" then
        error(sformat("gpu_transformer: optimizer '%s' is not supported (use 'adamw' or 'sgd')", opt), 2)
    end
    self.optimizer    = opt
    local dt = string.lower(tostring(cfg.dtype or "f32"))
    self.dtype        = (dt == "bf16" or dt == "bfloat16") and luaTL.BF16 or luaTL.F32
    self.decode_batch = cfg.decode_batch or 1
    self.N            = self.B * self.T
    self.attn_scale   = 1.0 / sqrt(self.hd)
    self.steps        = 0
    self.freed        = false

    self.h = lm.create{ vocab = self.vocab, dim = self.dim, layers = self.layers, heads = self.heads,
                        ffn = self.ffn, max_seq = self.T, batch = self.B, decode_batch = self.decode_batch,
                        tie = self.tie, dtype = self.dtype, use_rope = self.use_rope, causal = self.causal,
                        rope_interleaved = cfg.rope_interleaved, kv_splits = cfg.kv_splits,
                        eps = self.eps, rope_base = self.rope_base }

    -- parameter table in the reference's order: tok_emb, {ln1, wqkv, wo, ln2, w13, w2} x L, lnf [, head] (:224-239)
    self.params = {}
    local name = ffi.new("char[32]")
    local r, c, dec, off = ffi.new("int32_t[1]"), ffi.new("int32_t[1]"), ffi.new("int32_t[1]"), ffi.new("int64_t[1]")
    for i = 0, C.luaTL_lm_ntensors(self.h) - 1 do
        lm.check(C.luaTL_lm_tensor_info(self.h, i, name, r, c, off, dec), "lm.tensor_info")
        self.params[#self.params + 1] = { name = ffi.string(name), rows = r[0], cols = c[0], nelem = r[0] * c[0],
                                          offset = tonumber(off[0]), decay = dec[0] ~= 0 }
    end

    -- host staging: static [B, T] id / target blocks, the result and argument structs, one logits row
    self.h_ids  = ffi.new("int32_t[?]", self.N)
    self.h_tgt  = ffi.new("int32_t[?]", self.N)
    self.res    = ffi.new("luaTL_lm_result_t")
    self.args   = ffi.new("luaTL_lm_train_args_t")
    self.args.optimizer    = (opt == "sgd") and 0 or 1
    self.args.weight_decay = self.weight_decay
    self.args.clip_norm    = self.clip_norm
    self.args.beta1, self.args.beta2, self.args.adam_eps = self.beta1, self.beta2, self.adam_eps
    self._row   = ffi.new("float[?]", self.vocab)
    self._last_ms = -1

    -- fp32 model on the tensor cores (TF32 products, 2e-3 instead of 1e-4)
    if cfg.tf32 then lm.check(C.luaTL_lm_set_tf32(self.h, 1), "lm.set_tf32") end
    if cfg.init ~= false then self:_init_weights(cfg.seed) end
    return self
end

--- GPT-2 style init of the reference (:85-98, :217-239): N(0, 0.02) by Box-Muller, wo and w2 scaled by 1/sqrt(2L),
--- gains 1.  Streams through write_param in 64 Ki-element chunks.
function Model:_init_weights(seed)
    if seed then math.randomseed(seed) end
    local CH = 65536
    local buf = ffi.new("float[?]", CH)
    local rscale = 1.0 / sqrt(2 * self.layers)
    for i = 1, #self.params do
        local p = self.params[i]
        local is_gain = (p.rows == 1)
        local scale = 0.02
        if p.name:find("%.wo$") or p.name:find("%.w2$") then scale = 0.02 * rscale end
        local done = 0
        while done < p.nelem do
            local n = math.min(CH, p.nelem - done)
            for k = 0, n - 1 do
                if is_gain then
                    buf[k] = 1.0
                else
                    local u1, u2 = math.random(), math.random()
                    if u1 < 1e-12 then u1 = 1e-12 end
                    buf[k] = scale * sqrt(-2.0 * math.log(u1)) * math.cos(2.0 * math.pi * u2)
                end
            end
            self:write_param(i, done + 1, n, buf)
            done = done + n
        end
    end
end

--- Pack up to B windows {inp, tgt, n} of 1-indexed ids into the static blocks (pad: id 0, target -1).  Returns the
--- number of valid targets.  Same contract and error text as the reference (:567-605).
function Model:_pack(windows, nwin)
    local B, T, V = self.B, self.T, self.vocab
    local ib, tb = self.h_ids, self.h_tgt
    local valid = 0
    for b = 0, B - 1 do
        local base = b * T
        local w = (b < (nwin or B)) and windows[b + 1] or nil
        local n = 0
        if w then
            local inp, tgt = w[1], w[2]
            n = w[3] or #inp
            if n > T then n = T end
            for t = 0, n - 1 do
                local a, y = inp[t + 1], tgt[t + 1]
                if a < 1 or a > V or y < 1 or y > V then
                    error(sformat("gpu_transformer: token out of range at window %d, pos %d " ..
                          "(input %s, target %s, vocab %d)", b + 1, t + 1, tostring(a), tostring(y), V), 3)
                end
                ib[base + t] = a - 1
                tb[base + t] = y - 1
            end
            valid = valid + n
        end
        for t = n, T - 1 do
            ib[base + t] = 0
            tb[base + t] = -1
        end
    end
    return valid
end

--- One optimizer step over up to B windows.  Returns loss, correct, valid, grad_norm, finite (:637-661).
function Model:train_step(windows, nwin, lr, step)
    if self.freed then error("gpu_transformer: train_step() on a freed model", 2) end
    local valid = self:_pack(windows, nwin)
    local a = self.args
    a.lr, a.step = lr, step or (self.steps + 1)
    a.valid_global, a.no_update, a.accumulate, a.skip_allreduce = 0, 0, 0, 0
    lm.check(C.luaTL_lm_train_step(self.h, self.h_ids, self.h_tgt, a, self.res), "lm.train_step")
    local r = self.res
    self._last_ms = r.step_ms
    local finite = r.finite ~= 0
    if finite then self.steps = self.steps + 1 end
    return r.loss, r.correct, valid, r.grad_norm, finite
end

--- Forward-only loss / accuracy (:664-669).
function Model:eval_step(windows, nwin)
    if self.freed then error("gpu_transformer: eval_step() on a freed model", 2) end
    local valid = self:_pack(windows, nwin)
    lm.check(C.luaTL_lm_eval_step(self.h, self.h_ids, self.h_tgt, self.res), "lm.eval_step")
    return self.res.loss, self.res.correct, valid
end

local function row_proxy(buf, V, base)
    return setmetatable({}, { __index = function(_, i)
        local j = i - base
        if j < 1 or j > V then
            error("gpu_transformer: forward() materializes only the final row of the logits (index " ..
                  tostring(i) .. " is outside it)", 2)
        end
        return buf[j - 1]
    end })
end

--- Duck-typed forward for the cache-less branch of LMTrain:generate (:677-708): last logits row only.
function Model:forward(ids)
    local T, V = self.T, self.vocab
    local n = #ids
    if n < 1 then error("gpu_transformer: forward() needs at least one token", 2) end
    local first = 1
    if n > T then first, n = n - T + 1, T end
    for t = 0, n - 1 do
        local a = ids[first + t]
        if a < 1 or a > V then
            error(sformat("gpu_transformer: token out of range at pos %d (input %s, vocab %d)", t + 1, tostring(a), V), 2)
        end
        self.h_ids[t] = a - 1
    end
    lm.check(C.luaTL_lm_forward(self.h, self.h_ids, 1, n, self._row, 1), "lm.forward")
    return { data = { rows = n, cols = V, data = row_proxy(self._row, V, (n - 1) * V) } }
end

--- KV-cache state of one sequence (ai/nn/transformer.lua:284): slot = which cache line of decode_batch it uses.
function Model:new_state(slot)
    slot = slot or 0
    lm.check(C.luaTL_lm_slot_reset(self.h, slot), "lm.slot_reset")
    return { n = 0, slot = slot }
end

--- Feed one token (1-indexed) to the sequence, append its K/V, return the logits row as a 1-indexed proxy
--- (ai/nn/transformer.lua:297).  A full context raises, as the CPU model's step does; generate() then re-prefills.
function Model:step(id, state)
    if id < 1 or id > self.vocab then
        error(sformat("gpu_transformer: step() token %s outside 1..%d", tostring(id), self.vocab), 2)
    end
    lm.check(C.luaTL_lm_step(self.h, state.slot, id - 1, self._row), "lm.step")
    state.n = state.n + 1
    return { data = { rows = 1, cols = self.vocab, data = row_proxy(self._row, self.vocab, 0) } }
end

function Model:prefill(ids, state)
    local out
    for i = 1, #ids do out = self:step(ids[i], state) end
    return out
end

--- Batched generation on the device: prompts = array of equally long arrays of 1-indexed ids; returns an array of
--- arrays with n_new ids each.  Greedy unless set_sampling gave a temperature.
function Model:generate_batch(prompts, n_new)
    local nseq, npr = #prompts, #prompts[1]
    local p = ffi.new("int32_t[?]", nseq * npr)
    for b = 1, nseq do
        if #prompts[b] ~= npr then error("gpu_transformer: generate_batch() needs prompts of one length", 2) end
        for t = 1, npr do p[(b - 1) * npr + t - 1] = prompts[b][t] - 1 end
    end
    local out = ffi.new("int32_t[?]", nseq * n_new)
    lm.check(C.luaTL_lm_generate(self.h, p, nseq, npr, n_new, out, self.res), "lm.generate")
    self._last_ms = self.res.step_ms
    local res = {}
    for b = 1, nseq do
        local row = {}
        for t = 1, n_new do row[t] = out[(b - 1) * n_new + t - 1] + 1 end
        res[b] = row
    end
    return res
end

--- temperature <= 0: greedy.  top_k / top_p as in pick_token (ai/optim/lmtrain.lua:1364-1436); stop_id 1-indexed.
function Model:set_sampling(o)
    o = o or {}
    lm.check(C.luaTL_lm_set_sampling(self.h, o.temperature or 0, o.top_k or 0, o.top_p or 0, o.seed or 0,
                                     o.stop_id and (o.stop_id - 1) or -1), "lm.set_sampling")
end

--- Capture fwd+bwd as a CUDA graph (:714-728): the native step replays it while the valid-target count is the one
--- it was captured with (:643) and captures again when it changes.
function Model:capture()
    if self.graph_on then return true end
    lm.check(C.luaTL_lm_set_graph(self.h, 1), "lm.set_graph")
    self.graph_on = true
    return true
end

function Model:maybe_capture()
    if self.use_graph and not self.graph_on and (self.steps or 0) >= 2 then self:capture() end
    self.graph_ready = C.luaTL_lm_graph_ready(self.h) ~= 0
end

--- Device-to-device snapshot of the weights into one flat buffer (:746-794); pass the previous one back to reuse it.
function Model:snapshot(reuse)
    if self.freed then error("gpu_transformer: snapshot() on a freed model", 2) end
    local snap = reuse
    if snap and snap.owner ~= self then self:release_snapshot(snap); snap = nil end
    if not snap then snap = { owner = self, buf = adapter.alloc(1, self:nparams()) } end
    lm.check(C.luaTL_gpu_copy(C.luaTL_lm_params_device(self.h), ffi.cast("float*", snap.buf.t.data), self:nparams()),
             "snapshot copy")
    return snap
end

function Model:restore(snap)
    if not snap then return false end
    if self.freed then error("gpu_transformer: restore() on a freed model", 2) end
    if snap.owner ~= nil and snap.owner ~= self then
        error("gpu_transformer: restore() was handed a snapshot taken from a different model instance", 2)
    end
    lm.check(C.luaTL_gpu_copy(ffi.cast("float*", snap.buf.t.data), C.luaTL_lm_params_device(self.h), self:nparams()),
             "restore copy")
    return true
end

function Model:release_snapshot(snap)
    if type(snap) ~= "table" then return false end
    if snap.buf and snap.buf.free then pcall(function() snap.buf:free() end) end
    snap.buf, snap.owner = nil, nil
    return true
end

--- Stream elements [from, from+count-1] (1-indexed) of parameter i into the 0-indexed float buffer dst (:799-811).
function Model:read_param(i, from, count, dst)
    if self.freed then error("gpu_transformer: read_param() on a freed model", 2) end
    local p = self.params[i]
    if not p then error(sformat("gpu_transformer: no parameter %d", i), 2) end
    if from < 1 or (from + count - 1) > p.nelem then
        error(sformat("gpu_transformer: read_param range %d..%d outside parameter %d (%d elems)",
              from, from + count - 1, i, p.nelem), 2)
    end
    lm.check(C.luaTL_lm_read_params(self.h, p.offset + from - 1, count, dst), "param.download")
    return count
end

--- Inverse of read_param (:813-829).
function Model:write_param(i, from, count, src)
    if self.freed then error("gpu_transformer: write_param() on a freed model", 2) end
    local p = self.params[i]
    if not p then error(sformat("gpu_transformer: no parameter %d", i), 2) end
    if from < 1 or (from + count - 1) > p.nelem then
        error(sformat("gpu_transformer: write_param range %d..%d outside parameter %d (%d elems)",
              from, from + count - 1, i, p.nelem), 2)
    end
    lm.check(C.luaTL_lm_write_params(self.h, p.offset + from - 1, count, src), "param.upload")
    return count
end

function Model:free()
    if self.freed then return end
    self.freed = true
    lm.destroy(self.h)
    self.h, self.params, self.graph_ready = nil, {}, false
end

function Model:parameters() return self.params end

function Model:nparams()
    return tonumber(C.luaTL_lm_nparams(self.h))
end

--- FLOPs of one fwd+bwd step by the reference's model (:860-873): 3 x forward GEMM FLOPs, full T x T attention.
function Model:flops_per_step()
    local B, T, D, H, hd = self.B, self.T, self.dim, self.heads, self.hd
    local F, V, L, N = self.ffn, self.vocab, self.layers, self.N
    local f = L * (2 * N * (3 * D) * D + 2 * B * H * (2 * T * T * hd) + 2 * N * D * D + 2 * N * (2 * F) * D + 2 * N * D * F)
    f = f + 2 * N * V * D
    return 3 * f, f
end

function Model:vram()
    local free, total = luaTL.mem_info()
    local st = luaTL.pool_stats()
    return { free = free, total = total, pool_in_use = st.in_use, pool_reserved = st.reserved, pool_peak = st.peak }
end

function Model:last_step_ms()
    return self._last_ms
end

return GT
