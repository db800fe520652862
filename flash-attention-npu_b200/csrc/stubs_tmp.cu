#include "fa_internal.h"
namespace fa {
}
extern "C" {
int fa_mla_decode(const fa_mla_params*) { return fa::fail(FA_ERR_UNSUPPORTED, "n/a"); }
size_t fa_mla_workspace_bytes(const fa_mla_params*) { return 0; }
int fa_mla_num_splits(const fa_mla_params*) { return 1; }
}
