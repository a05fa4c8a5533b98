// Pipeline schedules (1F1B and interleaved), an in-process multi-stage executor that runs
// them over mailboxes, tensor-parallel linear forwards and the DP x TP x PP rank arithmetic.
// Reference surface: include/cg_pipeline.h, src/pipeline/{pipeline,tensor_parallel}.c.
// The multi-GPU executor of the same schedules lives in the Python package (NCCL p2p).
#include <map>
#include <tuple>

#include "internal.hpp"

using namespace cgi;

namespace {
struct Impl {
  // (kind 0 = activation / 1 = gradient, destination stage, micro-batch) -> tensor
  std::map<std::tuple<int, int, int>, cg_tensor*> mail;
  int loss_kind = 0;
  ~Impl() { for (auto& kv : mail) cg_tensor_release(kv.second); }
};
Impl* impl_of(cg_pipeline_parallel* pp) { return (Impl*)pp->impl; }
void push(std::vector<cg_schedule_step>& v, cg_schedule_action a, int mb, int stage) { v.push_back({a, mb, stage}); }
void fwd_steps(std::vector<cg_schedule_step>& v, int mb, int stage, int first, int last, int tag) {
  if (stage != first) push(v, SCHEDULE_RECV_FWD, mb, tag);
  push(v, SCHEDULE_FORWARD, mb, tag);
  if (stage != last) push(v, SCHEDULE_SEND_FWD, mb, tag);
}
void bwd_steps(std::vector<cg_schedule_step>& v, int mb, int stage, int first, int last, int tag) {
  if (stage != last) push(v, SCHEDULE_RECV_BWD, mb, tag);
  push(v, SCHEDULE_BACKWARD, mb, tag);
  if (stage != first) push(v, SCHEDULE_SEND_BWD, mb, tag);
}
cg_schedule_step* to_c(const std::vector<cg_schedule_step>& v, int* len) {
  cg_schedule_step* out = (cg_schedule_step*)std::malloc(sizeof(cg_schedule_step) * (v.size() ? v.size() : 1));
  std::copy(v.begin(), v.end(), out);
  if (len) *len = (int)v.size();
  return out;
}
}  // namespace

// One stage's 1F1B program: S-1-stage warm-up forwards, then one forward / one backward in
// alternation, then the remaining backwards, then the optimizer.  At most S-stage
// micro-batches are in flight on a stage.
CG_EXPORT cg_schedule_step* cg_pipeline_gen_1f1b_stage(int S, int M, int stage, int* len) {
  if (S <= 0 || M <= 0 || stage < 0 || stage >= S) { if (len) *len = 0; return fail(CG_ERROR_INVALID_ARGUMENT, (cg_schedule_step*)nullptr); }
  std::vector<cg_schedule_step> v;
  const int warm = S - 1 - stage < M ? S - 1 - stage : M;
  int f = 0, b = 0;
  for (; f < warm; ++f) fwd_steps(v, f, stage, 0, S - 1, stage);
  for (; f < M; ++f) { fwd_steps(v, f, stage, 0, S - 1, stage); bwd_steps(v, b, stage, 0, S - 1, stage); ++b; }
  for (; b < M; ++b) bwd_steps(v, b, stage, 0, S - 1, stage);
  push(v, SCHEDULE_OPTIMIZER, -1, stage);
  return to_c(v, len);
}
CG_EXPORT cg_schedule_step* cg_pipeline_gen_1f1b(int S, int M, int* len) { return cg_pipeline_gen_1f1b_stage(S, M, 0, len); }

// Interleaved 1F1B for pipeline rank `rank` holding V model chunks (virtual stage = chunk * S +
// rank, carried in stage_id).  M must be a multiple of S.
CG_EXPORT cg_schedule_step* cg_pipeline_gen_interleaved_stage(int S, int V, int M, int rank, int* len) {
  if (S <= 0 || V <= 0 || M <= 0 || rank < 0 || rank >= S || M % S) { if (len) *len = 0; return fail(CG_ERROR_INVALID_ARGUMENT, (cg_schedule_step*)nullptr); }
  const int total = M * V, last_virtual = S * V - 1;
  int warm = (S - rank - 1) * 2 + (V - 1) * S;
  if (warm > total) warm = total;
  auto chunk_of = [&](int k, bool fwd) { const int c = (k / S) % V; return fwd ? c : V - 1 - c; };
  auto mb_of = [&](int k) { return (k / (S * V)) * S + k % S; };
  std::vector<cg_schedule_step> v;
  int f = 0, b = 0;
  auto do_f = [&]() { const int vs = chunk_of(f, true) * S + rank; fwd_steps(v, mb_of(f), vs, 0, last_virtual, vs); ++f; };
  auto do_b = [&]() { const int vs = chunk_of(b, false) * S + rank; bwd_steps(v, mb_of(b), vs, 0, last_virtual, vs); ++b; };
  while (f < warm) do_f();
  while (f < total) { do_f(); do_b(); }
  while (b < total) do_b();
  push(v, SCHEDULE_OPTIMIZER, -1, rank);
  return to_c(v, len);
}
CG_EXPORT cg_schedule_step* cg_pipeline_gen_interleaved(int S, int V, int M, int* len) { return cg_pipeline_gen_interleaved_stage(S, V, M, 0, len); }

CG_EXPORT cg_pipeline_parallel* cg_pipeline_new(int S, int M) {
  if (S <= 0 || M <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_pipeline_parallel*)nullptr);
  cg_pipeline_parallel* pp = (cg_pipeline_parallel*)std::calloc(1, sizeof(cg_pipeline_parallel));
  pp->num_stages = S; pp->num_microbatches = M;
  pp->stages = (cg_pipeline_stage*)std::calloc(S, sizeof(cg_pipeline_stage));
  for (int s = 0; s < S; ++s) pp->stages[s].stage_id = s;
  pp->schedule = cg_pipeline_gen_1f1b(S, M, &pp->schedule_len);
  pp->impl = new Impl();
  return pp;
}
CG_EXPORT void cg_pipeline_set_stage(cg_pipeline_parallel* pp, int stage, void* layers, int num_layers) {
  if (!pp || stage < 0 || stage >= pp->num_stages) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  pp->stages[stage].layers = layers; pp->stages[stage].num_layers = num_layers;
}
// 0: mean-squared error (default); 1: softmax cross-entropy against one-hot targets
CG_EXPORT void cg_pipeline_set_loss(cg_pipeline_parallel* pp, int kind) { if (pp) impl_of(pp)->loss_kind = kind; }
CG_EXPORT void cg_pipeline_free(cg_pipeline_parallel* pp) {
  if (!pp) return;
  delete impl_of(pp);
  std::free(pp->stages); std::free(pp->schedule); std::free(pp);
}

static void mail_put(cg_pipeline_parallel* pp, int kind, int dest, int mb, const float* src, const cg_tensor* like) {
  cg_tensor* t = make_like(like, kind == 0);
  std::memcpy(t->data, src, sizeof(float) * t->size);
  auto key = std::make_tuple(kind, dest, mb);
  auto& slot = impl_of(pp)->mail[key];
  if (slot) cg_tensor_release(slot);
  slot = t;
}
static cg_tensor* mail_take(cg_pipeline_parallel* pp, int kind, int dest, int mb) {
  auto& mail = impl_of(pp)->mail;
  auto it = mail.find(std::make_tuple(kind, dest, mb));
  if (it == mail.end()) return nullptr;
  cg_tensor* t = it->second;
  mail.erase(it);
  return t;
}
CG_EXPORT void cg_pipeline_send_activation(cg_pipeline_parallel* pp, int dest, cg_tensor* a, int mb) {
  if (!pp || !a || dest < 0 || dest >= pp->num_stages) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  mail_put(pp, 0, dest, mb, a->data, a);
}
CG_EXPORT void cg_pipeline_send_gradient(cg_pipeline_parallel* pp, int dest, cg_tensor* g, int mb) {
  if (!pp || !g || dest < 0 || dest >= pp->num_stages) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  mail_put(pp, 1, dest, mb, g->grad ? g->grad : g->data, g);
}
static void recv_into(cg_pipeline_parallel* pp, int kind, int dest, cg_tensor* buf, int mb) {
  if (!pp || !buf) { set_error(CG_ERROR_NULL_POINTER); return; }
  cg_tensor* t = mail_take(pp, kind, dest, mb);
  if (!t) { set_error(CG_ERROR_TIMEOUT); return; }            // nothing was sent
  if (t->size != buf->size) set_error(CG_ERROR_SHAPE_MISMATCH);
  else std::memcpy(buf->data, t->data, sizeof(float) * t->size);
  cg_tensor_release(t);
}
CG_EXPORT void cg_pipeline_recv_activation(cg_pipeline_parallel* pp, int src, cg_tensor* buf, int mb) { recv_into(pp, 0, src + 1, buf, mb); }
CG_EXPORT void cg_pipeline_recv_gradient(cg_pipeline_parallel* pp, int src, cg_tensor* buf, int mb) { recv_into(pp, 1, src - 1, buf, mb); }

// Runs every stage's 1F1B program in one process: a stage advances whenever the message its
// next step waits for has arrived.  input / target are split along dimension 0 into
// num_microbatches equal parts; parameter gradients accumulate the mean over micro-batches.
CG_EXPORT void cg_pipeline_forward_backward(cg_pipeline_parallel* pp, cg_tensor* input, cg_tensor* target) {
  if (!pp || !input || !target) { set_error(CG_ERROR_NULL_POINTER); return; }
  const int S = pp->num_stages, M = pp->num_microbatches;
  for (int s = 0; s < S; ++s) if (!pp->stages[s].layers) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  if (input->ndim < 1 || input->shape[0] % M || target->shape[0] != input->shape[0]) { set_error(CG_ERROR_SHAPE_MISMATCH); return; }
  const int mbs = input->shape[0] / M;
  pp->global_batch_size = input->shape[0]; pp->micro_batch_size = mbs;
  auto slice = [&](cg_tensor* t, int m, bool rg) {
    int shape[CG_MAX_DIMS];
    for (int i = 0; i < t->ndim; ++i) shape[i] = t->shape[i];
    shape[0] = mbs;
    cg_tensor* o = make(shape, t->ndim, rg);
    std::memcpy(o->data, t->data + (size_t)m * o->size, sizeof(float) * o->size);
    return o;
  };
  std::vector<std::vector<cg_schedule_step>> prog(S);
  for (int s = 0; s < S; ++s) { int n; cg_schedule_step* p = cg_pipeline_gen_1f1b_stage(S, M, s, &n); prog[s].assign(p, p + n); std::free(p); }
  std::vector<size_t> pc(S, 0);
  // per (stage, micro-batch): received input, produced output, loss, received gradient
  std::vector<std::vector<cg_tensor*>> in(S, std::vector<cg_tensor*>(M, nullptr)), out = in, loss = in, gin = in;
  double loss_sum = 0;
  bool progress = true, failed = false;
  while (progress && !failed) {
    progress = false;
    for (int s = 0; s < S && !failed; ++s) {
      while (pc[s] < prog[s].size()) {
        const cg_schedule_step st = prog[s][pc[s]];
        const int m = st.microbatch_id;
        if (st.action == SCHEDULE_RECV_FWD) { cg_tensor* t = mail_take(pp, 0, s, m); if (!t) break; in[s][m] = t; }
        else if (st.action == SCHEDULE_RECV_BWD) { cg_tensor* t = mail_take(pp, 1, s, m); if (!t) break; gin[s][m] = t; }
        else if (st.action == SCHEDULE_FORWARD) {
          if (s == 0) in[s][m] = slice(input, m, false);
          cg_tensor* y = cg_sequential_forward((cg_sequential*)pp->stages[s].layers, in[s][m]);
          if (!y) { failed = true; break; }
          out[s][m] = y;                                   // ours: the stage handed us a reference
          if (s == S - 1) {
            cg_tensor* tm = slice(target, m, false);
            loss[s][m] = impl_of(pp)->loss_kind == 1 ? cg_softmax_cross_entropy_loss(y, tm, CG_REDUCTION_MEAN) : cg_mse_loss(y, tm, CG_REDUCTION_MEAN);
            cg_tensor_release(tm);
            if (!loss[s][m]) { failed = true; break; }
            loss_sum += loss[s][m]->data[0];
          }
        } else if (st.action == SCHEDULE_SEND_FWD) mail_put(pp, 0, s + 1, m, out[s][m]->data, out[s][m]);
        else if (st.action == SCHEDULE_BACKWARD) {
          if (s == S - 1) { ensure_grad(loss[s][m]); loss[s][m]->grad[0] = 1.0f / M; cg_backward(loss[s][m]); }
          else { ensure_grad(out[s][m]); std::memcpy(out[s][m]->grad, gin[s][m]->data, sizeof(float) * out[s][m]->size); cg_backward(out[s][m]); }
        } else if (st.action == SCHEDULE_SEND_BWD) mail_put(pp, 1, s - 1, m, in[s][m]->grad, in[s][m]);
        ++pc[s]; progress = true;
      }
    }
  }
  for (int s = 0; s < S; ++s) {
    if (pc[s] != prog[s].size()) failed = true;              // a stage is stuck: the schedule deadlocked
    for (int m = 0; m < M; ++m) for (cg_tensor* t : {in[s][m], out[s][m], loss[s][m], gin[s][m]}) if (t) cg_tensor_release(t);
  }
  pp->last_loss = (float)(loss_sum / M);
  if (failed) set_error(CG_ERROR_TIMEOUT);
}
// Averages parameter gradients over the data-parallel group.  One process is the whole group
// here, so the mean is the identity; multi-process groups reduce in the Python package.
CG_EXPORT void cg_pipeline_allreduce_grads(cg_pipeline_parallel* pp) {
  if (!pp) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (pp->dp_group && pp->dp_group->world_size > 1) set_error(CG_ERROR_INVALID_ARGUMENT);
}

// ---------------------------------------------------------- tensor parallel
// weight is this rank's shard.  Column-parallel: Y_shard = X @ W[:, shard]; row-parallel:
// partial Y = X[:, shard] @ W[shard, :], to be summed over the group.  With a one-rank group
// both are the complete result.
static cg_tensor* tp_matmul(cg_tensor* x, cg_tensor* w) {
  if (!x || !w) return fail(CG_ERROR_NULL_POINTER, (cg_tensor*)nullptr);
  if (w->ndim != 2 || cols_of(x) != w->shape[0]) return fail(CG_ERROR_SHAPE_MISMATCH, (cg_tensor*)nullptr);
  return cg_matmul(x, w);
}
CG_EXPORT cg_tensor* cg_tp_column_parallel_forward(cg_tensor_parallel_linear* tp, cg_tensor* x, cg_tensor* w) { (void)tp; return tp_matmul(x, w); }
CG_EXPORT cg_tensor* cg_tp_row_parallel_forward(cg_tensor_parallel_linear* tp, cg_tensor* x, cg_tensor* w) { (void)tp; return tp_matmul(x, w); }

// ------------------------------------------------------------- 3-D layout
// world rank r: tp = r % TP, pp = (r / TP) % PP, dp = r / (TP * PP)  (src/pipeline/pipeline.c).
static cg_distributed_group* new_group(cg_parallel_mode mode, int size) {
  cg_distributed_group* g = (cg_distributed_group*)std::calloc(1, sizeof(cg_distributed_group));
  g->mode = mode; g->world_size = size; g->ranks = (int*)std::calloc(size, sizeof(int));
  return g;
}
static void free_group(cg_distributed_group* g) { if (g) { std::free(g->ranks); std::free(g); } }
CG_EXPORT cg_3d_parallel* cg_3d_parallel_new(int dp, int tp, int pp) {
  if (dp <= 0 || tp <= 0 || pp <= 0) return fail(CG_ERROR_INVALID_ARGUMENT, (cg_3d_parallel*)nullptr);
  cg_3d_parallel* c = (cg_3d_parallel*)std::calloc(1, sizeof(cg_3d_parallel));
  c->dp_size = dp; c->tp_size = tp; c->pp_size = pp; c->world_size = dp * tp * pp;
  c->dp_group = new_group(PARALLEL_DATA, dp); c->tp_group = new_group(PARALLEL_TENSOR, tp); c->pp_group = new_group(PARALLEL_PIPELINE, pp);
  cg_3d_parallel_init_from_world(c, c->world_size, 0);
  return c;
}
CG_EXPORT void cg_3d_parallel_init_from_world(cg_3d_parallel* c, int world, int rank) {
  if (!c) { set_error(CG_ERROR_NULL_POINTER); return; }
  if (world != c->dp_size * c->tp_size * c->pp_size || rank < 0 || rank >= world) { set_error(CG_ERROR_INVALID_ARGUMENT); return; }
  const int TP = c->tp_size, PP = c->pp_size;
  c->world_size = world; c->world_rank = rank;
  c->tp_rank = rank % TP; c->pp_rank = (rank / TP) % PP; c->dp_rank = rank / (TP * PP);
  auto rank_of = [&](int d, int p, int t) { return (d * PP + p) * TP + t; };
  for (int i = 0; i < c->tp_size; ++i) c->tp_group->ranks[i] = rank_of(c->dp_rank, c->pp_rank, i);
  for (int i = 0; i < c->pp_size; ++i) c->pp_group->ranks[i] = rank_of(c->dp_rank, i, c->tp_rank);
  for (int i = 0; i < c->dp_size; ++i) c->dp_group->ranks[i] = rank_of(i, c->pp_rank, c->tp_rank);
  c->tp_group->rank = c->tp_rank; c->pp_group->rank = c->pp_rank; c->dp_group->rank = c->dp_rank;
}
CG_EXPORT void cg_3d_parallel_free(cg_3d_parallel* c) {
  if (!c) return;
  free_group(c->dp_group); free_group(c->tp_group); free_group(c->pp_group); std::free(c);
}
