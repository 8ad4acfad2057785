-- luaTL_lm: LuaJIT binding of the fused, device-resident language model of luaTL.so for B200.
--
-- Load after the reference's own bindings (ai/gpu/luaTL.lua, ai/gpu/luaTL_train.lua): they cdef the op-level
-- surface and load the shared library; this file only adds the declarations of the new entry points
-- (include/luatl_b200.h, "fused device-resident model" and "data-parallel gradient exchange") and a handful of
-- helpers.  Types are spelled exactly as in the header; tests parse this block and the header and compare.
--
--   package.path = "lua/?.lua;" .. package.path     -- ahead of the reference's ai/gpu/?.lua
--   local lm = require("luaTL_lm")
local ffi   = require("ffi")
local luaTL = require("luaTL")          -- the reference's binding: structs, ck(), ffi.load
require("luaTL_train")                   -- its train surface (fails loudly on a core-only library)

ffi.cdef[[
typedef struct {
    int32_t vocab, dim, layers, heads, ffn;
    int32_t max_seq;
    int32_t batch;
    int32_t decode_batch;
    int32_t tie;
    int32_t dtype;
    int32_t use_rope, rope_interleaved, causal;
    int32_t kv_splits;
    float   eps, rope_base;
} luaTL_lm_config_t;

typedef struct {
    float   loss;
    float   grad_norm;
    int32_t correct, valid, finite;
    float   step_ms;
} luaTL_lm_result_t;

typedef struct {
    int32_t optimizer, step;
    float   lr, weight_decay, clip_norm, beta1, beta2, adam_eps;
    int32_t valid_global;
    int32_t no_update;
    int32_t accumulate;
    int32_t skip_allreduce;
} luaTL_lm_train_args_t;

typedef struct luaTL_lm_s luaTL_lm_t;

luaTL_lm_t* luaTL_lm_create(const luaTL_lm_config_t* cfg);
void        luaTL_lm_destroy(luaTL_lm_t* m);
int64_t luaTL_lm_nparams(const luaTL_lm_t* m);
int     luaTL_lm_ntensors(const luaTL_lm_t* m);
int     luaTL_lm_tensor_info(const luaTL_lm_t* m, int i, char* name32, int32_t* rows, int32_t* cols,
                             int64_t* offset, int32_t* decay);
int luaTL_lm_write_params(luaTL_lm_t* m, int64_t offset, int64_t count, const float* host);
int luaTL_lm_read_params(luaTL_lm_t* m, int64_t offset, int64_t count, float* host);
int luaTL_lm_read_grads(luaTL_lm_t* m, int64_t offset, int64_t count, float* host);
float* luaTL_lm_params_device(luaTL_lm_t* m);
float* luaTL_lm_grads_device(luaTL_lm_t* m);
int luaTL_lm_train_step(luaTL_lm_t* m, const int32_t* ids, const int32_t* targets,
                        const luaTL_lm_train_args_t* a, luaTL_lm_result_t* out);
int luaTL_lm_train_step_dev(luaTL_lm_t* m, const int32_t* d_ids, const int32_t* d_targets,
                            const luaTL_lm_train_args_t* a, luaTL_lm_result_t* out);
int luaTL_lm_set_tf32(luaTL_lm_t* m, int on);
int luaTL_lm_set_graph(luaTL_lm_t* m, int on);
int luaTL_lm_graph_ready(const luaTL_lm_t* m);
int luaTL_lm_eval_step(luaTL_lm_t* m, const int32_t* ids, const int32_t* targets, luaTL_lm_result_t* out);
int luaTL_lm_forward(luaTL_lm_t* m, const int32_t* ids, int nseq, int ntok, float* logits_host, int last_only);
int luaTL_lm_state_reset(luaTL_lm_t* m);
int luaTL_lm_slot_reset(luaTL_lm_t* m, int slot);
int luaTL_lm_step(luaTL_lm_t* m, int slot, int32_t id, float* logits_host);
int luaTL_lm_state_len(luaTL_lm_t* m, int slot);
int luaTL_lm_generate(luaTL_lm_t* m, const int32_t* prompts, int nseq, int n_prompt, int n_new,
                      int32_t* out, luaTL_lm_result_t* timing);
int luaTL_lm_generate_dev(luaTL_lm_t* m, const int32_t* d_prompts, int nseq, int n_prompt, int n_new,
                          int32_t* d_out, luaTL_lm_result_t* timing);
int luaTL_lm_set_sampling(luaTL_lm_t* m, float temperature, int top_k, float top_p, uint64_t seed, int stop_id);
int luaTL_lm_last_timing(luaTL_lm_t* m, float* prefill_ms, float* decode_ms, int64_t* launches);
int luaTL_sgd(float* w, const float* g, uint64_t n, float lr, float wd, const float* nsq, float max_norm);
int luaTL_sample_rows(const float* logits, int rows, int vocab, float temperature, int top_k, float top_p, uint64_t seed,
                      const int32_t* counters, int32_t* out);
int luaTL_comm_unique_id(char* id128);
int luaTL_comm_init(const char* id128, int world, int rank);
int luaTL_comm_world(void);
int luaTL_comm_allreduce_f32(float* dev, uint64_t n);
void luaTL_comm_destroy(void);
]]

local M = {}
M.C = luaTL.C

--- Raise with the library's message on a non-zero status (same text as the reference's ck(), ai/gpu/luaTL.lua:240-246).
function M.check(status, ctx)
    return luaTL.check(status, ctx)
end

--- New model handle from a plain table (see gpu_transformer.lua for the field meaning); freed by the GC or M.destroy.
function M.create(cfg)
    local c = ffi.new("luaTL_lm_config_t")
    c.vocab, c.dim, c.layers, c.heads, c.ffn = cfg.vocab, cfg.dim, cfg.layers, cfg.heads, cfg.ffn
    c.max_seq, c.batch, c.decode_batch = cfg.max_seq, cfg.batch or 1, cfg.decode_batch or 1
    c.tie = (cfg.tie == false) and 0 or 1
    c.dtype = cfg.dtype or luaTL.F32
    c.use_rope = (cfg.use_rope == false) and 0 or 1
    c.rope_interleaved = cfg.rope_interleaved and 1 or 0
    c.causal = (cfg.causal == false) and 0 or 1
    c.kv_splits = cfg.kv_splits or 0
    c.eps, c.rope_base = cfg.eps or 1e-5, cfg.rope_base or 10000
    local h = M.C.luaTL_lm_create(c)
    if h == nil then
        error("luaTL[lm_create]: " .. ffi.string(M.C.luaTL_get_last_error()), 2)
    end
    return ffi.gc(h, M.C.luaTL_lm_destroy)
end

function M.destroy(h)
    if h ~= nil then M.C.luaTL_lm_destroy(ffi.gc(h, nil)) end
end

return M
