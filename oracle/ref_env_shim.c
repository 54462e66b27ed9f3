/*
 * Record producer built from the reference's own C environment (TEST
 * INFRASTRUCTURE; compiled only where the reference sources are present).
 *
 * The reference's craftax_full.c keeps every function static and carries a
 * main(); this translation unit includes it unmodified (path given with
 * -DCFX_REF_C=\"...\") with CRAFTAX_COMPACT_OBS defined, so that the
 * environment's observation buffer IS the [n][996] compact record array
 * (craftax_full.c:2956-2958), and exports thin wrappers around its batched
 * harness (cf_vec_init craftax_full.c:8276, c_step, cf_xorshift32 :8238).
 */
#define CRAFTAX_COMPACT_OBS 1
#define main cf_ref_main
#include CFX_REF_C
#undef main

typedef struct { CfVec v; } refenv;

void* refenv_create(int num_envs, unsigned long long seed) {
    refenv* r = (refenv*)calloc(1, sizeof(refenv));
    cf_vec_init(&r->v, num_envs, (uint64_t)seed, /*parallel=*/1);
    return r;
}

void refenv_destroy(void* h) {
    refenv* r = (refenv*)h;
    cf_vec_free(&r->v);
    free(r);
}

int refenv_record_size(void) { return (int)CRAFTAX_OBS_SIZE; }
int refenv_num_actions(void) { return (int)CRAFTAX_NUM_ACTIONS; }

/* One step with the harness's own per-env xorshift action stream
 * (craftax_full.c:8350-8353). */
void refenv_step_random(void* h) {
    refenv* r = (refenv*)h;
    CfVec* v = &r->v;
    #pragma omp parallel for schedule(static)
    for (int i = 0; i < v->num_envs; i++) {
        v->actions[i] = (float)(cf_xorshift32(&v->action_rng[i]) % CRAFTAX_NUM_ACTIONS);
        c_step(&v->envs[i]);
    }
}

/* One step with caller-provided actions (float-coded, as the env reads them). */
void refenv_step(void* h, const float* actions) {
    refenv* r = (refenv*)h;
    CfVec* v = &r->v;
    #pragma omp parallel for schedule(static)
    for (int i = 0; i < v->num_envs; i++) {
        v->actions[i] = actions[i];
        c_step(&v->envs[i]);
    }
}

const unsigned char* refenv_records(void* h) { return (const unsigned char*)((refenv*)h)->v.observations; }
const float* refenv_terminals(void* h) { return ((refenv*)h)->v.terminals; }
const float* refenv_rewards(void* h) { return ((refenv*)h)->v.rewards; }
const float* refenv_actions(void* h) { return ((refenv*)h)->v.actions; }
