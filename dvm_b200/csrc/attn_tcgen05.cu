// placeholder
#include "mm_launch.h"
namespace dvmb {
int LaunchAttention(const AttnParam &, void *) { return -1; }
bool AttentionSupported(const AttnParam &) { return false; }
unsigned int ReadAttentionStatus() { return 0; }
}
