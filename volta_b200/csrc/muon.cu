// Placeholder until the Muon path lands: every entry reports VB_ERR_UNSUPPORTED.
#include "engine.h"

namespace vb {
struct MuonState {};
void destroy_muon_state(MuonState *s) { delete s; }
int muon_init(vb_optimizer *) { return fail(VB_ERR_UNSUPPORTED, "Muon is not built yet"); }
int muon_step(vb_optimizer *, uint32_t) { return fail(VB_ERR_UNSUPPORTED, "Muon is not built yet"); }
int muon_download_update(vb_optimizer *, int64_t, float *, int64_t) { return fail(VB_ERR_UNSUPPORTED, "Muon is not built yet"); }
int muon_last_flops(vb_optimizer *, double *) { return fail(VB_ERR_UNSUPPORTED, "Muon is not built yet"); }
int muon_owner(vb_optimizer *, int64_t) { return 0; }
}  // namespace vb
