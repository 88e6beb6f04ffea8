// Link check only: pulls in the reference engine's Transformer and Model so that every
// ternary:: operator they call must be resolved by libtllm_b200.so.  Never run.
#include "transformer.h"
#include "model.h"

int main(int argc, char**)
{
    if (argc > 1000) {            // never true; keeps the objects referenced
        Model m;
        Transformer t(m);
        t.reset();
        return t.forward(nullptr, 1, 0) != nullptr;
    }
    return 0;
}
