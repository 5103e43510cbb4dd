/* TEST INFRASTRUCTURE ONLY — never linked into, loaded by or called from the product library.
 *
 * The segment planner of the reference (plan_segments / plan_segments_vad / find_split_point,
 * src/mynah_asr.c:1177-1323) is file-static, so this shim includes that translation unit as it
 * is and forwards to it; the Silero VAD (src/vad.c) is public and forwarded directly. No
 * arithmetic lives here. */
#include "mynah_asr.c"

mynah_asr_vad *ref_vad_open(const char *dir) { return mynah_asr_vad_open(dir); }
void ref_vad_close(mynah_asr_vad *v) { mynah_asr_vad_close(v); }
void ref_vad_reset(mynah_asr_vad *v) { mynah_asr_vad_reset(v); }
float ref_vad_feed(mynah_asr_vad *v, const float *samples, size_t n) { return mynah_asr_vad_feed(v, samples, n); }

/* spans as pairs of sample offsets: out[2i], out[2i+1] */
int ref_vad_speech_spans(mynah_asr_vad *v, const float *samples, size_t n, long long *out, int cap) {
    mynah_asr_vad_span *s = malloc((size_t)(cap > 0 ? cap : 1) * sizeof(*s));
    if (!s) return -1;
    const int k = mynah_asr_vad_speech_spans(v, samples, n, s, cap);
    for (int i = 0; i < k; i++) { out[2 * i] = (long long)s[i].t0; out[2 * i + 1] = (long long)s[i].t1; }
    free(s);
    return k;
}

/* plan_segments on a model that has only what the planner reads: the sample rate, the segment
 * limit and (optionally) a VAD. Segments as pairs offset, length. */
int ref_plan_segments(const float *samples, size_t n, int sample_rate, double seg_sec, mynah_asr_vad *vad,
                      long long *out, int cap) {
    struct mynah_asr_model *m = calloc(1, sizeof(*m));
    if (!m) return -1;
    m->feat.sample_rate = sample_rate;
    m->seg_sec = seg_sec;
    m->vad = vad;
    seg_range *segs = NULL;
    const int k = plan_segments(m, samples, n, &segs);
    for (int i = 0; i < k && i < cap; i++) { out[2 * i] = (long long)segs[i].off; out[2 * i + 1] = (long long)segs[i].len; }
    free(segs);
    free(m);
    return k;
}
