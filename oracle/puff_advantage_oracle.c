/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the V-trace-clipped GAE advantage
 * recurrence.  Nothing in the shipped package may link, import or execute this
 * file; only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg do, and there only as the checker / the timed CPU arm.
 *
 * Plain-C restatement of the reference CPU implementation
 *   pufferlib/extensions/pufferlib.cpp:28-41  (puff_advantage_row)
 *   pufferlib/extensions/pufferlib.cpp:63-72  (puff_advantage, row loop)
 *   pufferlib/extensions/pufferlib.cpp:43-59  (vtrace_check, argument rules)
 * The arithmetic keeps the reference's expression order and rounding: every
 * product and sum is an individually rounded fp32 operation (build with
 * -ffp-contract=off, no -ffast-math, no -mfma), and `1 - dones` is a double
 * subtraction narrowed to float exactly as the reference writes it.
 *
 * Parity is pinned: the build recipe next to this file compiles the reference
 * source itself into oracle/_ref/ and tests/test_oracle.py asserts bit
 * equality between the two on every benchmark configuration; the committed
 * fixtures under tests/golden/ were produced by that reference build.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

/* One [horizon] row, walked backwards.  advantages[horizon-1] is never
 * written (pufferlib.cpp:31: the loop starts at horizon-2). */
static void oracle_row(const float *values, const float *rewards,
                       const float *dones, const float *importance,
                       float *advantages, float gamma, float lambda,
                       float rho_clip, float c_clip, int64_t horizon)
{
    float last = 0.0f;
    for (int64_t t = horizon - 2; t >= 0; t--) {
        const int64_t tn = t + 1;
        /* pufferlib.cpp:34 -- `1.0 - dones[t_next]` is evaluated in double */
        const float nonterminal = (float)(1.0 - (double)dones[tn]);
        const float rho = fminf(importance[t], rho_clip);   /* :35 */
        const float c = fminf(importance[t], c_clip);       /* :36 */
        /* :37  rho*(r' + gamma*v'*nn - v), left-to-right */
        const float gv = gamma * values[tn];
        const float gvn = gv * nonterminal;
        const float td = (rewards[tn] + gvn) - values[t];
        const float delta = rho * td;
        /* :38  delta + gamma*lambda*c*last*nn, left-to-right */
        const float gl = gamma * lambda;
        const float glc = gl * c;
        const float glca = glc * last;
        const float carry = glca * nonterminal;
        last = delta + carry;
        advantages[t] = last;                               /* :39 */
    }
}

/* Row loop of pufferlib.cpp:63-72 with 64-bit offsets. */
void puff_oracle_advantage(const float *values, const float *rewards,
                           const float *dones, const float *importance,
                           float *advantages, float gamma, float lambda,
                           float rho_clip, float c_clip,
                           int64_t num_segments, int64_t horizon)
{
    for (int64_t s = 0; s < num_segments; s++) {
        const int64_t off = s * horizon;
        oracle_row(values + off, rewards + off, dones + off, importance + off,
                   advantages + off, gamma, lambda, rho_clip, c_clip, horizon);
    }
}

/* Per-segment sum of |advantage| over columns 0..horizon-2, accumulated in
 * double.  Stands in for `advantages.abs().sum(axis=1)` (pufferl.py:359) when
 * the caller passes a zero-filled buffer (pufferl.py:353), as a
 * high-precision checker for the fused epilogue. */
void puff_oracle_abs_sum(const float *advantages, double *abs_sum,
                         int64_t num_segments, int64_t horizon)
{
    for (int64_t s = 0; s < num_segments; s++) {
        double acc = 0.0;
        for (int64_t t = 0; t + 1 < horizon; t++)
            acc += fabs((double)advantages[s * horizon + t]);
        abs_sum[s] = acc;
    }
}

/* Prioritised-replay weights of pufferl.py:359-361 in double:
 *   w = nan_to_num(abs_sum ** alpha, 0, 0, 0);  p = (w + 1e-6)/(sum(w) + 1e-6)
 * `total_w` lets a sharded caller pass the all-reduced sum; pass a negative
 * value to use the local sum. Returns the local sum of w. */
double puff_oracle_priorities(const double *abs_sum, double *weights,
                              double *probs, double alpha, double total_w,
                              int64_t num_segments)
{
    double local = 0.0;
    for (int64_t s = 0; s < num_segments; s++) {
        double w = pow(abs_sum[s], alpha);
        if (isnan(w) || isinf(w)) w = 0.0;
        weights[s] = w;
        local += w;
    }
    const double denom = (total_w < 0.0 ? local : total_w) + 1e-6;
    if (probs)
        for (int64_t s = 0; s < num_segments; s++)
            probs[s] = (weights[s] + 1e-6) / denom;
    return local;
}

/* Minibatch gather and advantage normalisation of pufferl.py:363, 373-375,
 * 408-409 in double:
 *   mb_prio = (num_segments * prio_probs[idx]) ** -beta
 *   mb_values = values[idx]; mb_returns = advantages[idx] + mb_values
 *   adv_norm = mb_prio * (adv - mean(adv)) / (std(adv) + 1e-8),  unbiased std
 * over all gathered elements (torch.std default). */
void puff_oracle_minibatch(const float *advantages, const float *values,
                           const double *prio_probs, const int64_t *idx,
                           double *mb_values, double *mb_returns,
                           double *mb_adv_norm, double *mb_prio, double beta,
                           int64_t num_segments, int64_t horizon,
                           int64_t mb_segments)
{
    const double n = (double)mb_segments * (double)horizon;
    double sum = 0.0;
    for (int64_t m = 0; m < mb_segments; m++)
        for (int64_t t = 0; t < horizon; t++)
            sum += (double)advantages[idx[m] * horizon + t];
    const double mean = sum / n;
    double ss = 0.0;
    for (int64_t m = 0; m < mb_segments; m++)
        for (int64_t t = 0; t < horizon; t++) {
            const double d = (double)advantages[idx[m] * horizon + t] - mean;
            ss += d * d;
        }
    const double std = sqrt(ss / (n - 1.0));
    for (int64_t m = 0; m < mb_segments; m++) {
        const double prio = pow((double)num_segments * prio_probs[idx[m]], -beta);
        mb_prio[m] = prio;
        for (int64_t t = 0; t < horizon; t++) {
            const double a = (double)advantages[idx[m] * horizon + t];
            const double v = (double)values[idx[m] * horizon + t];
            mb_values[m * horizon + t] = v;
            mb_returns[m * horizon + t] = a + v;
            mb_adv_norm[m * horizon + t] = prio * (a - mean) / (std + 1e-8);
        }
    }
}
